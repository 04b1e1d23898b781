// torch.classes.dgs_classes.BlockPipeline: mini-batches in flight.
//
// The reference overlaps the sampling of the next mini-batches with the work on
// the current one through DGL's DataLoader wrapped around ChunkTensorSampler
// (oppo_bench/single_node/chunktensor.py:120-172, utils/chunktensor_sampler.py:63-118);
// inside one batch its operators still stop at every size read-back.  This class
// is that loader's role in native form, without DGL: `depth` slots, each with its
// own CUDA stream, pinned size / status words, workspace and output buffers that
// are allocated once for the largest batch.  submit(seeds) queues the whole
// multi-hop sample + relabel sequence (dgs_sample_blocks) and, when a feature
// table was given, the feature gather of the resulting input nodes directly behind
// it (dgs_gather_rows_counted takes the row count from the device), all on the
// slot's stream and without the host reading anything back.  next() hands out the
// oldest batch: it waits for that batch's sizes (normally there already), makes
// the caller's current stream wait for the slot's stream, and returns views of the
// slot's buffers.  With two or more batches submitted ahead, the latency-bound
// kernels of one batch's small hops run while another batch's gather keeps the
// memory system (HBM, NVLink, host link) busy.
//
// Lifetime of the results: views into the slot, valid until the submit() that
// takes the slot again (the depth-th submit() after the one that queued the
// batch).  That submit() first makes the slot's stream wait for everything queued
// so far on the caller's current stream, so consumers that were launched there
// before it are safe.
//
// The twenty driver calls that queue a batch (about 60-80 us of host time) are made
// by a thread the pipeline owns: submit() only fixes what must happen on the
// caller's thread (the ordering event on its stream, the random stream of the
// batch) and hands the rest over, so the caller's thread -- in the reference's
// setting the Python training loop -- is free again after a few microseconds.
// next() waits for that thread to have queued the batch before it waits for the
// batch's sizes.  Failures of the queuing calls are kept and thrown by next().
// The launches of the sampling sequence are the same for every batch of a slot
// that has the same number of seeds, so a slot records them once
// (dgs_sample_blocks_record) and later batches replay the recording with one
// call; the random stream of a batch travels through two pinned words.
// DGS_PIPELINE_RECORD=0 keeps every batch on individual launches.
//
// No counterpart in src/pybind.cc: an addition like the _CAPI_sample_blocks*
// operators, built from the same C ABI calls.
#pragma once
#include <ATen/cuda/CUDAGeneratorImpl.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <string>
#include <thread>

#include "chunk_tensor.h"

namespace dgs {

// (seed, offset) from torch's default CUDA generator, so torch.manual_seed
// controls sampling; a call that needs `streams` independent random streams uses
// offset, offset + 1, ... and the generator moves past them.
inline std::pair<uint64_t, uint64_t> next_rng(uint64_t streams = 1) {
  auto gen = at::get_generator_or_default<at::CUDAGeneratorImpl>(
      c10::nullopt, at::cuda::detail::getDefaultCUDAGenerator());
  std::lock_guard<std::mutex> lock(gen->mutex_);
  const uint64_t seed = gen->current_seed();
  const uint64_t offset = gen->get_offset();
  gen->set_offset(offset + 4 * ((streams + 3) / 4));  // torch keeps the offset a multiple of 4
  return {seed, offset};
}

using PipelineResult = std::tuple<torch::Tensor, std::vector<torch::Tensor>, std::vector<torch::Tensor>,
                                  std::vector<int64_t>, torch::Tensor>;

class BlockPipeline : public torch::CustomClassHolder {
 public:
  BlockPipeline(c10::intrusive_ptr<ChunkTensor> indptr, c10::intrusive_ptr<ChunkTensor> indices,
                c10::optional<c10::intrusive_ptr<ChunkTensor>> probs,
                c10::optional<c10::intrusive_ptr<ChunkTensor>> features, std::vector<int64_t> fanouts,
                bool replace, int64_t max_seeds, int64_t depth, int64_t src_nodes)
      : indptr_(std::move(indptr)), indices_(std::move(indices)), replace_(replace), max_seeds_(max_seeds) {
    if (probs.has_value() && probs.value().defined()) probs_ = probs.value();
    if (features.has_value() && features.value().defined()) features_ = features.value();
    H_ = static_cast<int>(fanouts.size());
    TORCH_CHECK(H_ >= 1 && H_ <= DGS_MAX_HOPS, "BlockPipeline: between 1 and ", DGS_MAX_HOPS, " fan-outs");
    TORCH_CHECK(max_seeds >= 1, "BlockPipeline: max_seeds must be >= 1");
    TORCH_CHECK(depth >= 1 && depth <= 16, "BlockPipeline: depth must be in 1..16");
    for (int64_t k : fanouts) TORCH_CHECK(k >= 1, "BlockPipeline: fan-outs must be >= 1");
    TORCH_CHECK(indptr_->dtype() == indices_->dtype() &&
                    (indptr_->dtype() == torch::kInt64 || indptr_->dtype() == torch::kInt32),
                "BlockPipeline: indptr and indices must share one id type (int32 or int64)");
    TORCH_CHECK(!probs_.defined() || probs_->dtype() == torch::kFloat, "probs must be float32");
    ids64_ = indptr_->dtype() == torch::kInt64;
    device_ = indptr_->device();
    // A frontier cannot hold more distinct ids than the id space has.  That space is indptr's node count
    // unless the caller says that `indices` holds ids of a larger one (a bipartite CSC): src_nodes.
    TORCH_CHECK(src_nodes >= 0, "BlockPipeline: src_nodes must be >= 0 (0: the node count of indptr)");
    id_space_ = std::max<int64_t>(indptr_->desc().total - 1, src_nodes);
    // the reference applies the fan-outs last to first (chunktensor_sampler.py:97)
    applied_.assign(fanouts.rbegin(), fanouts.rend());

    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
    dgs_hop hops[DGS_MAX_HOPS];
    DGS_CHECK_RC(dgs_sample_blocks_bounds(max_seeds_, applied_.data(), H_, id_space_, hops));
    ws_bytes_ = dgs_sample_blocks_workspace_bytes(hops, H_);
    const int64_t esz = ids64_ ? 8 : 4;
    int64_t slot_bytes = static_cast<int64_t>(ws_bytes_) + max_seeds_ * esz;
    for (int h = 0; h < H_; ++h) {
      edge_cap_[h] = hops[h].seed_bound * hops[h].fanout;
      frontier_cap_[h] = hops[h].frontier_bound;
      slot_bytes += (2 * edge_cap_[h] + frontier_cap_[h]) * esz;
    }
    if (features_.defined())
      slot_bytes += frontier_cap_[H_ - 1] * features_->elem_stride() * static_cast<int64_t>(dtype_size(features_->dtype()));
    TORCH_CHECK(slot_bytes * depth <= kBudgetBytes, "BlockPipeline: ", depth, " slots of ", slot_bytes,
                " bytes exceed the ", kBudgetBytes, "-byte budget; lower max_seeds, the fan-outs or depth");

    const auto dev = torch::Device(torch::kCUDA, static_cast<c10::DeviceIndex>(device_));
    const auto id_opt = torch::TensorOptions().dtype(indptr_->dtype()).device(dev);
    slots_ = std::vector<Slot>(static_cast<size_t>(depth));
    // The sampling sequence is a chain of short kernels with thousands of CTAs each; the feature gather is one
    // long kernel that, in its bulk-copy form, needs a single small CTA per SM for its whole duration and
    // keeps its bytes in flight in shared memory.  Each slot therefore gathers on a stream of its own with the
    // HIGHER priority: the gather's few CTAs are placed as soon as an SM has room and then stay out of the
    // way, while the sampling kernels of the other batches keep filling the rest of every SM.  (Measured on the
    // Products-shaped step, three batches deep: 0.146 ms; with the priorities the other way round 0.148 ms,
    // with everything of a batch on one stream 0.147 ms.)
    int prio_low = 0, prio_high = 0;
    TORCH_CHECK(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high) == cudaSuccess,
                "BlockPipeline: cannot query stream priorities");
    for (Slot& s : slots_) {
      TORCH_CHECK(cudaStreamCreateWithPriority(&s.stream, cudaStreamNonBlocking, prio_low) == cudaSuccess,
                  "BlockPipeline: cannot create a stream");
      if (features_.defined())
        TORCH_CHECK(cudaStreamCreateWithPriority(&s.gather_stream, cudaStreamNonBlocking, prio_high) == cudaSuccess,
                    "BlockPipeline: cannot create a stream");
      TORCH_CHECK(cudaEventCreateWithFlags(&s.ready, cudaEventDisableTiming) == cudaSuccess &&
                      cudaEventCreateWithFlags(&s.sampled, cudaEventDisableTiming) == cudaSuccess &&
                      cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming) == cudaSuccess,
                  "BlockPipeline: cannot create an event");
      void* p = nullptr;
      TORCH_CHECK(cudaHostAlloc(&p, 256, cudaHostAllocPortable | cudaHostAllocMapped) == cudaSuccess,
                  "BlockPipeline: cannot allocate pinned words");
      std::memset(p, 0, 256);
      s.sizes = static_cast<int64_t*>(p);
      s.status = reinterpret_cast<int32_t*>(static_cast<char*>(p) + 2 * DGS_MAX_HOPS * sizeof(int64_t));
      s.rng_words = reinterpret_cast<uint64_t*>(static_cast<char*>(p) + 192);
      s.seeds = torch::empty({max_seeds_}, id_opt);
      s.ws = byte_scratch(ws_bytes_, dev);
      for (int h = 0; h < H_; ++h) {
        s.rows.push_back(torch::empty({edge_cap_[h]}, id_opt));
        s.cols.push_back(torch::empty({edge_cap_[h]}, id_opt));
        s.frontier.push_back(torch::empty({frontier_cap_[h]}, id_opt));
      }
      if (features_.defined())
        s.feats = torch::empty({frontier_cap_[H_ - 1], features_->elem_stride()},
                               torch::TensorOptions().dtype(features_->dtype()).device(dev));
    }
    // the buffers were allocated on the current stream; nothing of theirs is pending there, but make the
    // slots' streams start after whatever the allocator's stream still holds
    TORCH_CHECK(cudaStreamSynchronize(current_stream()) == cudaSuccess, "BlockPipeline: synchronisation failed");
    static const char* record_env = std::getenv("DGS_PIPELINE_RECORD");
    record_ = !(record_env != nullptr && record_env[0] == '0');
    static const char* inline_env = std::getenv("DGS_PIPELINE_INLINE_SUBMIT");  // 1: queue on the caller's thread
    if (!(inline_env != nullptr && inline_env[0] == '1')) worker_ = std::thread([this] { worker_loop(); });
  }

  ~BlockPipeline() override {
    if (worker_.joinable()) {
      {
        std::lock_guard<std::mutex> lock(mu_);
        stop_ = true;
      }
      cv_.notify_all();
      worker_.join();
    }
    for (Slot& s : slots_) {
      if (s.stream != nullptr) cudaStreamSynchronize(s.stream);
      if (s.gather_stream != nullptr) cudaStreamSynchronize(s.gather_stream);
      dgs_sample_blocks_recording_free(s.recording);
      if (s.ready != nullptr) cudaEventDestroy(s.ready);
      if (s.sampled != nullptr) cudaEventDestroy(s.sampled);
      if (s.done != nullptr) cudaEventDestroy(s.done);
      if (s.stream != nullptr) cudaStreamDestroy(s.stream);
      if (s.gather_stream != nullptr) cudaStreamDestroy(s.gather_stream);
      if (s.sizes != nullptr) cudaFreeHost(s.sizes);
    }
  }

  // Queue one mini-batch.  `seeds`: 1-D ids of the graph's id type, at most max_seeds of them, on the
  // pipeline's device or in (preferably pinned) host memory; they are copied into the slot ON THE CALLER'S
  // CURRENT STREAM, so whatever the caller does with its tensor afterwards on that stream (overwrite it,
  // free it) is ordered behind the copy.
  void submit(torch::Tensor seeds) {
    TORCH_CHECK(in_flight_ < static_cast<int64_t>(slots_.size()),
                "BlockPipeline.submit: all ", slots_.size(), " slots hold batches; call next() first");
    TORCH_CHECK(seeds.scalar_type() == indptr_->dtype(), "seeds, indptr and indices must share one id type");
    TORCH_CHECK(seeds.device().is_cpu() || (seeds.device().is_cuda() && seeds.device().index() == device_),
                "BlockPipeline.submit: seeds must be on the pipeline's device or on the host");
    seeds = seeds.contiguous().view({-1});
    const int64_t n = seeds.numel();
    TORCH_CHECK(n <= max_seeds_, "BlockPipeline.submit: ", n, " seeds, the pipeline was built for ", max_seeds_);
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
    Slot& s = slots_[head_ % slots_.size()];
    report_late_status(s, "BlockPipeline.submit");
    s.n_seeds = n;
    s.batch = head_;
    s.error.clear();
    if (n > 0) {
      // the seeds go into the slot on the caller's stream; then everything the caller queued so far (the
      // seeds' producer, this copy, consumers of the slot's previous results) comes before the slot's own
      // stream: the event is recorded here, on the caller's thread and stream
      const size_t esz = ids64_ ? 8 : 4;
      TORCH_CHECK(cudaMemcpyAsync(s.seeds.data_ptr(), seeds.data_ptr(), n * esz,
                                  seeds.device().is_cpu() ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice,
                                  current_stream()) == cudaSuccess,
                  "BlockPipeline.submit: copying the seeds failed: ", cudaGetErrorString(cudaGetLastError()));
      TORCH_CHECK(cudaEventRecord(s.ready, current_stream()) == cudaSuccess,
                  "BlockPipeline.submit: cannot record an event on the current stream");
      for (int h = 0; h < H_; ++h) s.sizes[2 * h] = s.sizes[2 * h + 1] = kPending;
      Job job;
      job.slot = static_cast<int>(head_ % slots_.size());
      job.rng = next_rng(static_cast<uint64_t>(H_));
      if (worker_.joinable()) {
        s.state.store(kQueuing, std::memory_order_release);
        {
          std::lock_guard<std::mutex> lock(mu_);
          jobs_.push_back(std::move(job));
        }
        cv_.notify_one();
      } else {
        queue_batch(job);
        TORCH_CHECK(s.error.empty(), s.error);
      }
    }
    ++head_;
    ++in_flight_;
  }

  // The oldest submitted batch: (input_nodes, coo_rows, coo_cols, [n_src_0, n_dst_0, n_src_1, ...], features)
  // with the blocks in layer order, outermost hop first, exactly as _CAPI_sample_blocks* returns them;
  // features is [len(input_nodes), D] (empty when the pipeline has no feature table).
  PipelineResult next() {
    TORCH_CHECK(in_flight_ > 0, "BlockPipeline.next: nothing was submitted");
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
    Slot& s = slots_[tail_ % slots_.size()];
    std::vector<torch::Tensor> rows(H_), cols(H_);
    std::vector<int64_t> shape(2 * H_);
    torch::Tensor frontier, feats;
    int64_t n_dst = s.n_seeds;
    if (s.n_seeds == 0) {
      for (int h = 0; h < H_; ++h) {
        rows[h] = s.rows[0].narrow(0, 0, 0);
        cols[h] = s.cols[0].narrow(0, 0, 0);
      }
      frontier = s.frontier[0].narrow(0, 0, 0);
      if (features_.defined()) feats = s.feats.narrow(0, 0, 0);
    } else {
      // the submitting thread must have queued the batch (recorded `done`) before anything can wait for it
      for (uint64_t spins = 1; s.state.load(std::memory_order_acquire) == kQueuing; ++spins) {
        if ((spins & 0x3F) == 0) std::this_thread::yield();
      }
      if (!s.error.empty()) {
        const std::string msg = s.error;
        s.error.clear();
        ++tail_;
        --in_flight_;
        TORCH_CHECK(false, msg);
      }
      for (int h = 0; h < H_; ++h) {
        const int64_t nnz = wait_size(s.sizes + 2 * h, s.stream, "BlockPipeline.next");
        const int64_t nu = wait_size(s.sizes + 2 * h + 1, s.stream, "BlockPipeline.next");
        TORCH_CHECK(nnz >= 0 && nnz <= s.edge_bound[h] && nu >= 0, "dgs: BlockPipeline returned an impossible size");
        if (nu > s.frontier_bound[h]) {
          // more distinct ids than the id space was said to have: the frontier was cut off
          cudaEventSynchronize(s.done);
          *s.status = 0;
          ++tail_;
          --in_flight_;
          TORCH_CHECK(false, "dgs: BlockPipeline batch ", s.batch, ": hop ", h, " found ", nu, " distinct ids, more than the ",
                      s.frontier_bound[h], " the id space allows; if `indices` holds ids beyond indptr's node count "
                      "(a bipartite graph), pass that id space as src_nodes");
        }
        const int at = H_ - 1 - h;
        rows[at] = s.rows[h].narrow(0, 0, nnz);
        cols[at] = s.cols[h].narrow(0, 0, nnz);
        shape[2 * at] = std::min(nu, s.frontier_bound[h]);
        shape[2 * at + 1] = n_dst;
        n_dst = shape[2 * at];
      }
      if (strict_status())
        TORCH_CHECK(cudaEventSynchronize(s.done) == cudaSuccess, "BlockPipeline.next: synchronisation failed");
      const int32_t st = *static_cast<volatile int32_t*>(s.status);
      if (st != 0) {
        *s.status = 0;
        ++tail_;
        --in_flight_;
        TORCH_CHECK(false, "dgs: BlockPipeline batch ", s.batch, ": a kernel reported ", status_text(st), " (code ",
                    st, ")");
      }
      // the caller's stream sees the batch complete (sampling, relabelling and the feature gather)
      TORCH_CHECK(cudaStreamWaitEvent(current_stream(), s.done, 0) == cudaSuccess,
                  "BlockPipeline.next: cannot order the current stream after the slot's stream");
      frontier = s.frontier[H_ - 1].narrow(0, 0, n_dst);
      if (features_.defined()) feats = s.feats.narrow(0, 0, n_dst);
    }
    if (!feats.defined()) feats = torch::empty({0}, torch::TensorOptions().dtype(torch::kFloat).device(frontier.device()));
    ++tail_;
    --in_flight_;
    return std::make_tuple(frontier, rows, cols, shape, feats);
  }

  int64_t pending() const { return in_flight_; }
  // slots whose sampling sequence is currently held as a recording (call with nothing in flight)
  int64_t recorded_slots() const {
    int64_t n = 0;
    for (const Slot& s : slots_) n += s.recording != nullptr ? 1 : 0;
    return n;
  }
  int64_t depth() const { return static_cast<int64_t>(slots_.size()); }

 private:
  static constexpr int64_t kBudgetBytes = int64_t(32) << 30;
  static constexpr int kIdle = 0, kQueuing = 1;

  struct Job {
    int slot = 0;
    std::pair<uint64_t, uint64_t> rng;
  };

  struct Slot {
    std::atomic<int> state{kIdle};  // kQueuing while the submitting thread still has the batch's launches to make
    std::string error;              // what went wrong while queuing, thrown by next()
    cudaStream_t stream = nullptr;         // sampling sequence
    cudaStream_t gather_stream = nullptr;  // feature gather (higher priority); null: everything on `stream`
    cudaEvent_t ready = nullptr, sampled = nullptr, done = nullptr;
    int64_t* sizes = nullptr;   // [2 * DGS_MAX_HOPS], pinned
    int32_t* status = nullptr;  // pinned
    uint64_t* rng_words = nullptr;  // pinned (seed, offset) of the batch, read by a replayed recording
    dgs_blocks_recording* recording = nullptr;  // the sampling sequence for `recorded_seeds` seeds
    int64_t recorded_seeds = -1, odd_seeds = -1;
    torch::Tensor seeds, ws, feats;
    std::vector<torch::Tensor> rows, cols, frontier;  // indexed by hop of application
    int64_t edge_bound[DGS_MAX_HOPS] = {0}, frontier_bound[DGS_MAX_HOPS] = {0};
    int64_t n_seeds = 0, batch = -1;
  };

  void worker_loop() {
    cudaSetDevice(device_);
    for (;;) {
      Job job;
      {
        std::unique_lock<std::mutex> lock(mu_);
        cv_.wait(lock, [this] { return stop_ || !jobs_.empty(); });
        if (jobs_.empty()) return;  // stop requested and nothing left to queue
        job = std::move(jobs_.front());
        jobs_.pop_front();
      }
      queue_batch(job);
      slots_[job.slot].state.store(kIdle, std::memory_order_release);
    }
  }

  // The driver calls of one batch; any failure ends up in the slot's `error`.
  void queue_batch(const Job& job) {
    Slot& s = slots_[job.slot];
    try {
      const int64_t n = s.n_seeds;
      TORCH_CHECK(cudaStreamWaitEvent(s.stream, s.ready, 0) == cudaSuccess,
                  "BlockPipeline: cannot order the slot's stream after the caller's stream");
      dgs_hop hops[DGS_MAX_HOPS];
      DGS_CHECK_RC(dgs_sample_blocks_bounds(n, applied_.data(), H_, id_space_, hops));
      for (int h = 0; h < H_; ++h) {
        hops[h].coo_row = s.rows[h].data_ptr();
        hops[h].coo_col = s.cols[h].data_ptr();
        hops[h].frontier = s.frontier[h].data_ptr();
        s.edge_bound[h] = hops[h].seed_bound * hops[h].fanout;
        s.frontier_bound[h] = hops[h].frontier_bound;
      }
      const dgs_chunk_desc* probs = probs_.defined() ? &probs_->desc() : nullptr;
      if (record_ && s.recorded_seeds != n && (s.recording == nullptr || s.odd_seeds == n)) {
        // first batch of the slot, or a new batch size seen twice in a row: record the sequence for it
        dgs_sample_blocks_recording_free(s.recording);
        s.recording = nullptr;
        s.recorded_seeds = -1;
        const int rc = dgs_sample_blocks_record(&indptr_->desc(), &indices_->desc(), probs, s.seeds.data_ptr(), ids64_,
                                                hops, H_, replace_, s.rng_words, s.ws.data_ptr(), ws_bytes_, s.sizes,
                                                s.status, s.stream, &s.recording);
        if (rc == DGS_OK) {
          s.recorded_seeds = n;
        } else {
          // recording is an optimisation: say so once and go on with individual launches
          record_ = false;
          TORCH_WARN("dgs: BlockPipeline could not record its launch sequence (", dgs_last_error(),
                     "); batches are queued launch by launch");
        }
      }
      s.odd_seeds = (s.recorded_seeds == n) ? -1 : n;
      if (s.recording != nullptr && s.recorded_seeds == n) {
        s.rng_words[0] = job.rng.first;
        s.rng_words[1] = job.rng.second;
        DGS_CHECK_RC(dgs_sample_blocks_replay(s.recording, s.stream));
      } else {
        DGS_CHECK_RC(dgs_sample_blocks(&indptr_->desc(), &indices_->desc(), probs, s.seeds.data_ptr(), ids64_, hops, H_,
                                       replace_, job.rng.first, job.rng.second, s.ws.data_ptr(), ws_bytes_, s.sizes,
                                       s.status, s.stream));
      }
      cudaStream_t last = s.stream;
      if (features_.defined()) {
        const int64_t* n_dev = dgs_sample_blocks_frontier_count(hops, H_, s.ws.data_ptr());
        TORCH_CHECK(n_dev != nullptr, "BlockPipeline: no frontier count");
        if (s.gather_stream != nullptr) {
          TORCH_CHECK(cudaEventRecord(s.sampled, s.stream) == cudaSuccess &&
                          cudaStreamWaitEvent(s.gather_stream, s.sampled, 0) == cudaSuccess,
                      "BlockPipeline: cannot order the gather after the sampling sequence");
          last = s.gather_stream;
        }
        DGS_CHECK_RC(dgs_gather_rows_counted(&features_->desc(), s.frontier[H_ - 1].data_ptr(), ids64_,
                                             s.frontier_bound[H_ - 1], n_dev, features_->elem_stride(),
                                             s.feats.data_ptr(), s.status, last));
      }
      TORCH_CHECK(cudaEventRecord(s.done, last) == cudaSuccess, "BlockPipeline: cannot record an event");
    } catch (const std::exception& e) {
      s.error = std::string("dgs: BlockPipeline batch ") + std::to_string(s.batch) + ": " + e.what();
    }
  }

  // a status left by kernels that were still running when next() handed the batch out
  static void report_late_status(Slot& s, const char* where) {
    const int32_t st = *static_cast<volatile int32_t*>(s.status);
    if (st != 0) {
      *s.status = 0;
      TORCH_CHECK(false, "dgs: a kernel of BlockPipeline batch ", s.batch, " reported ", status_text(st), " (code ", st,
                  ") after next() had returned it; noticed in ", where);
    }
  }

  c10::intrusive_ptr<ChunkTensor> indptr_, indices_, probs_, features_;
  std::vector<int64_t> applied_;
  bool replace_ = false, ids64_ = true, record_ = true;
  int H_ = 0;
  int device_ = 0;
  int64_t max_seeds_ = 0, id_space_ = 0;
  size_t ws_bytes_ = 0;
  int64_t edge_cap_[DGS_MAX_HOPS] = {0}, frontier_cap_[DGS_MAX_HOPS] = {0};
  std::vector<Slot> slots_;
  int64_t head_ = 0, tail_ = 0, in_flight_ = 0;
  // the submitting thread and its queue
  std::thread worker_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Job> jobs_;
  bool stop_ = false;
};

}  // namespace dgs
