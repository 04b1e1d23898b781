// Pinned words the kernels write data-dependent sizes and their status into,
// handed out per operator call.
//
// The reference reads every size back with a blocking copy in the middle of an
// operator (src/cuda/rowwise_sampling.cu:147, src/cuda/tensor_reindex.cu:129) and
// traps the GPU on a bad id (device asserts).  Here a kernel early in the
// operator's sequence writes the size into pinned memory, the host picks it up as
// soon as it lands, and errors are recorded in a status word.  Every call leases
// its own words, so calls from several host threads, or on several streams, do
// not see each other's sizes or errors.
//
// Status semantics:
//   * an error raised by a kernel that has finished by the time the operator
//     learns its sizes is thrown by that operator call;
//   * an error raised later (kernels still running when the operator returns, or
//     operators that never wait, such as _CAPI_index) is thrown by the next dgs
//     operator call on the device that finds it, and the message names the
//     operator that caused it;
//   * DGS_STRICT_STATUS=1 makes every operator synchronise its stream and check
//     before it returns.
#pragma once
#include <c10/util/Exception.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../../include/dgs_b200.h"

namespace dgs {

constexpr int64_t kPending = INT64_MIN;  // "the kernel has not written this size yet"
constexpr int kWordsPerLease = 24;       // int64 sizes per lease (>= 2 * DGS_MAX_HOPS + split counts)
static_assert(2 * DGS_MAX_HOPS + 4 <= kWordsPerLease, "a lease must hold the sizes of a sample_blocks call");

inline const char* status_text(int32_t st) {
  return st == DGS_ERR_RANGE ? "an out-of-range id" : (st == DGS_ERR_TABLE_FULL ? "a full hash table" : "an error");
}

inline bool strict_status() {
  static const bool on = [] {
    const char* e = std::getenv("DGS_STRICT_STATUS");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}

class WordPool {
 public:
  struct Slot {
    int64_t* sizes = nullptr;   // [kWordsPerLease], pinned
    int32_t* status = nullptr;  // [1], pinned
    cudaEvent_t done = nullptr; // recorded when the lease ends: later kernels of the call may still write
    const char* op = "";        // operator that holds / last held the slot
    bool busy = false;          // leased right now
    bool fenced = false;        // `done` has been recorded at least once
  };

  // one pool per device; created on first use with that device current
  static WordPool& for_device(int device) {
    static std::mutex mu;
    static std::vector<WordPool*> pools;
    std::lock_guard<std::mutex> lock(mu);
    if (static_cast<size_t>(device) >= pools.size()) pools.resize(device + 1, nullptr);
    if (pools[device] == nullptr) pools[device] = new WordPool();
    return *pools[device];
  }

  // A free slot whose previous call has completely left the GPU.  A status that a call left behind after it
  // had returned is thrown here, naming the call it belongs to.
  Slot* acquire(const char* op) {
    std::lock_guard<std::mutex> lock(mu_);
    for (Slot* s : slots_) {
      if (s->busy) continue;
      const int32_t st = *static_cast<volatile int32_t*>(s->status);
      if (st != 0) {
        *s->status = 0;
        TORCH_CHECK(false, "dgs: a kernel of an earlier ", s->op, " call reported ", status_text(st), " (code ", st,
                    ") after that call had returned; noticed on entering ", op);
      }
    }
    // slots are reused in the order they were released, so the first candidate has normally left the GPU
    Slot* pick = nullptr;
    const size_t n = slots_.size();
    for (size_t i = 0; i < n && pick == nullptr; ++i) {
      Slot* s = slots_[(cursor_ + i) % n];
      if (s->busy) continue;
      if (s->fenced && cudaEventQuery(s->done) != cudaSuccess) {
        cudaGetLastError();  // cudaErrorNotReady is no error
        continue;
      }
      pick = s;
      cursor_ = (cursor_ + i + 1) % n;
    }
    if (pick == nullptr) pick = grow();
    pick->busy = true;
    pick->op = op;
    return pick;
  }

  // End of a lease: kernels queued on `stream` may still write the slot's words, so it is handed out again
  // only after they have run.
  void release(Slot* s, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(mu_);
    if (cudaEventRecord(s->done, stream) == cudaSuccess) s->fenced = true;
    else cudaGetLastError();
    s->busy = false;
  }

 private:
  Slot* grow() {
    constexpr int kBatch = 32;
    constexpr size_t kStride = 256;  // bytes per slot: 24 sizes + status, padded
    void* p = nullptr;
    TORCH_CHECK(cudaHostAlloc(&p, kBatch * kStride, cudaHostAllocPortable | cudaHostAllocMapped) == cudaSuccess,
                "dgs: cannot allocate pinned size / status words");
    std::memset(p, 0, kBatch * kStride);
    Slot* first = nullptr;
    for (int i = 0; i < kBatch; ++i) {
      Slot* s = new Slot();
      char* base = static_cast<char*>(p) + i * kStride;
      s->sizes = reinterpret_cast<int64_t*>(base);
      s->status = reinterpret_cast<int32_t*>(base + kWordsPerLease * sizeof(int64_t));
      TORCH_CHECK(cudaEventCreateWithFlags(&s->done, cudaEventDisableTiming) == cudaSuccess,
                  "dgs: cannot create an event");
      slots_.push_back(s);
      if (first == nullptr) first = s;
    }
    return first;
  }

  std::mutex mu_;
  std::vector<Slot*> slots_;
  size_t cursor_ = 0;
};

// RAII lease of one slot for the duration of an operator call.
class Lease {
 public:
  Lease(const char* op, int device, cudaStream_t stream)
      : pool_(WordPool::for_device(device)), slot_(pool_.acquire(op)), stream_(stream), op_(op) {}
  ~Lease() { pool_.release(slot_, stream_); }
  Lease(const Lease&) = delete;
  Lease& operator=(const Lease&) = delete;

  int64_t* sizes() const { return slot_->sizes; }
  int32_t* status() const { return slot_->status; }

  // throw if a kernel of this call has reported an error so far
  void check() const {
    const int32_t st = *static_cast<volatile int32_t*>(slot_->status);
    if (st != 0) {
      *slot_->status = 0;
      TORCH_CHECK(false, "dgs: ", op_, ": a kernel reported ", status_text(st), " (code ", st, ")");
    }
  }
  // operators that do not wait for anything: check only in strict mode (after a synchronisation)
  void finish() const {
    if (!strict_status()) return;
    TORCH_CHECK(cudaStreamSynchronize(stream_) == cudaSuccess, "dgs: ", op_, ": stream synchronisation failed");
    check();
  }

 private:
  WordPool& pool_;
  WordPool::Slot* slot_;
  cudaStream_t stream_;
  const char* op_;
};

// Spin until a kernel has overwritten kPending in a pinned word; a stream query is the way out if the
// stream died, so the host never waits for a value that cannot arrive.
inline int64_t wait_size(volatile int64_t* word, cudaStream_t stream, const char* where) {
  for (uint64_t spins = 1;; ++spins) {
    int64_t v = *word;
    if (v != kPending) return v;
    if ((spins & 0x3FF) == 0) {
      const cudaError_t q = cudaStreamQuery(stream);
      if (q == cudaSuccess) {
        v = *word;
        TORCH_CHECK(v != kPending, "dgs: ", where, ": the stream finished without reporting a size");
        return v;
      }
      TORCH_CHECK(q == cudaErrorNotReady, "dgs: ", where, ": CUDA error while waiting: ", cudaGetErrorString(q));
    }
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }
}

}  // namespace dgs
