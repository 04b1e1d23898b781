// Multi-hop sample -> relabel as ONE queued launch sequence.
//
// Replaces the loop of ChunkTensorSampler.sample_blocks (reference
// oppo_bench/single_node/utils/chunktensor_sampler.py:93-118), which for every
// hop calls the sampling operator (one blocking size read-back,
// src/cuda/rowwise_sampling.cu:147) and then the relabel operator (another one,
// src/cuda/tensor_reindex.cu:129) from Python, so the GPU idles between hops
// while the host learns each size and allocates the next output.
//
// Here the sizes never leave the device while the sequence runs: every kernel
// takes its item count as a device word written by its predecessor (Count),
// grids and buffers are sized by upper bounds the host can compute up front
// (hop h has at most seeds_h * (1 + fanout_h) frontier nodes, and never more
// than the graph has), and the actual sizes go to a caller-supplied (pinned)
// array that the host reads once, after everything is queued.
//
// Per hop: plan -> sample -> insert -> count -> number; the plan launch also
// carries, as extra CTAs, two jobs that depend on nothing it does: clearing the
// table this hop will fill and relabelling the COO of the hop before (whose
// numbering is complete by then).  The last hop's COO is relabelled by a launch
// of its own.  From the second hop on the seed list is a relabel's unique list,
// so a seed's relabelled id is its position and the sampler writes that directly;
// only the first hop (whose seeds the caller may repeat) looks its rows up.
#include <cstdlib>
#include <new>

#include "common.cuh"
#include "launchers.h"
#include "philox.cuh"

namespace dgs {
namespace {

constexpr size_t WS_ALIGN = 256;
inline size_t ws_align(size_t x) { return (x + WS_ALIGN - 1) / WS_ALIGN * WS_ALIGN; }

struct InitWords {
  int64_t* n0;
  int64_t n0_value;
  int n_tickets;
  unsigned int* tickets[2 * DGS_MAX_HOPS];
  // a recorded sequence takes its random stream from memory: (seed, offset) at rng_src, read by this
  // kernel on every replay and folded into one Philox key per hop for the sampling kernels behind it
  const uint64_t* rng_src;
  uint64_t* keys;
  int n_keys;
};

__global__ void blocks_init_kernel(const InitWords w) {
  pdl_enter();
  if (threadIdx.x == 0) *w.n0 = w.n0_value;
  if (threadIdx.x < w.n_tickets) *w.tickets[threadIdx.x] = 0u;
  if (w.rng_src != nullptr && threadIdx.x < w.n_keys) {
    const volatile uint64_t* src = w.rng_src;  // host-written words: no cached copy
    w.keys[threadIdx.x] = fold_rng_key(src[0], src[1] + static_cast<uint64_t>(threadIdx.x));
  }
}

__global__ void zero_sizes_kernel(int64_t* sizes, int n) {
  if (threadIdx.x < n) sizes[threadIdx.x] = 0;
}

int check_hops(const dgs_hop* hops, int32_t n_hops, const char* who) {
  DGS_REQUIRE(hops != nullptr && n_hops >= 1 && n_hops <= DGS_MAX_HOPS, DGS_ERR_INVALID,
              "%s: between 1 and %d hops", who, DGS_MAX_HOPS);
  for (int h = 0; h < n_hops; ++h) {
    DGS_REQUIRE(hops[h].fanout >= 1 && hops[h].seed_bound >= 0 && hops[h].frontier_bound >= 0, DGS_ERR_INVALID,
                "%s: hop %d: fanout %lld, bounds %lld / %lld", who, h, (long long)hops[h].fanout,
                (long long)hops[h].seed_bound, (long long)hops[h].frontier_bound);
    DGS_REQUIRE(hops[h].seed_bound * (1 + hops[h].fanout) < (1ll << 30), DGS_ERR_UNSUPPORTED,
                "%s: hop %d may produce %lld keys", who, h, (long long)(hops[h].seed_bound * (1 + hops[h].fanout)));
    DGS_REQUIRE(h == 0 || hops[h].seed_bound == hops[h - 1].frontier_bound, DGS_ERR_INVALID,
                "%s: hop %d: seed_bound must equal the previous hop's frontier_bound", who, h);
  }
  return DGS_OK;
}

}  // namespace
}  // namespace dgs

extern "C" int dgs_sample_blocks_bounds(int64_t n_seeds, const int64_t* fanouts, int32_t n_hops,
                                        int64_t num_nodes, dgs_hop* hops) {
  using namespace dgs;
  DGS_REQUIRE(fanouts != nullptr && hops != nullptr && n_hops >= 1 && n_hops <= DGS_MAX_HOPS && n_seeds >= 0 &&
                  num_nodes >= 0,
              DGS_ERR_INVALID, "dgs_sample_blocks_bounds: bad arguments");
  int64_t n = n_seeds;
  for (int h = 0; h < n_hops; ++h) {
    DGS_REQUIRE(fanouts[h] >= 1 && fanouts[h] < (1 << 20), DGS_ERR_INVALID, "dgs_sample_blocks_bounds: fanout %lld",
                (long long)fanouts[h]);
    hops[h].fanout = fanouts[h];
    hops[h].seed_bound = n;
    DGS_REQUIRE(n * (1 + fanouts[h]) < (1ll << 30), DGS_ERR_UNSUPPORTED,
                "dgs_sample_blocks_bounds: hop %d may produce %lld keys", h, (long long)(n * (1 + fanouts[h])));
    int64_t f = n * (1 + fanouts[h]);
    // a frontier of valid ids cannot be longer than the node list
    if (f > num_nodes) f = num_nodes > n ? num_nodes : n;
    hops[h].frontier_bound = f;
    n = f;
  }
  return DGS_OK;
}

extern "C" size_t dgs_sample_blocks_workspace_bytes(const dgs_hop* hops, int32_t n_hops) {
  using namespace dgs;
  if (hops == nullptr || n_hops < 1 || n_hops > DGS_MAX_HOPS) return 0;
  size_t total = WS_ALIGN;  // control words
  for (int h = 0; h < n_hops; ++h) {
    total += ws_align(dgs_sample_plan_bytes(hops[h].seed_bound));
    total += ws_align(dgs_relabel_table_bytes(hops[h].seed_bound * (1 + hops[h].fanout)));
  }
  return total;
}

extern "C" const int64_t* dgs_sample_blocks_frontier_count(const dgs_hop* hops, int32_t n_hops, void* workspace) {
  using namespace dgs;
  if (hops == nullptr || workspace == nullptr || n_hops < 1 || n_hops > DGS_MAX_HOPS) return nullptr;
  // same walk as the carving in dgs_sample_blocks: the word sits in the last hop's table
  char* p = static_cast<char*>(workspace) + WS_ALIGN;
  for (int h = 0; h < n_hops; ++h) {
    const int64_t key_bound = hops[h].seed_bound * (1 + hops[h].fanout);
    p += ws_align(dgs_sample_plan_bytes(hops[h].seed_bound));
    if (h == n_hops - 1) return unique_total(p, key_bound);
    p += ws_align(dgs_relabel_table_bytes(key_bound));
  }
  return nullptr;
}

namespace dgs {
namespace {

// Queues the whole sequence on `stream`.  rng_words == nullptr: the keys come from (rng_seed, rng_offset) as
// launch parameters; otherwise the first kernel reads (seed, offset) from rng_words when it RUNS.
int queue_blocks(const dgs_chunk_desc* indptr, const dgs_chunk_desc* indices, const dgs_chunk_desc* probs,
                 const void* seeds, int32_t ids64, const dgs_hop* hops, int32_t n_hops, int32_t replace,
                 uint64_t rng_seed, uint64_t rng_offset, const uint64_t* rng_words, void* workspace,
                 size_t workspace_bytes, int64_t* sizes, int32_t* status, dgs_stream_t stream) {
  int rc = validate_desc(indptr, "dgs_sample_blocks(indptr)");
  if (rc != DGS_OK) return rc;
  rc = validate_desc(indices, "dgs_sample_blocks(indices)");
  if (rc != DGS_OK) return rc;
  if (probs != nullptr) {
    rc = validate_desc(probs, "dgs_sample_blocks(probs)");
    if (rc != DGS_OK) return rc;
    DGS_REQUIRE(probs->esz == 4, DGS_ERR_UNSUPPORTED, "dgs_sample_blocks: weights must be fp32");
  }
  rc = check_hops(hops, n_hops, "dgs_sample_blocks");
  if (rc != DGS_OK) return rc;
  const int esz = ids64 ? 8 : 4;
  DGS_REQUIRE(indptr->esz == esz && indices->esz == esz, DGS_ERR_INVALID,
              "dgs_sample_blocks: indptr / indices element size does not match the id type");
  DGS_REQUIRE(sizes != nullptr, DGS_ERR_INVALID, "dgs_sample_blocks: null sizes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n0 = hops[0].seed_bound;
  if (n0 == 0) {
    zero_sizes_kernel<<<1, 32, 0, s>>>(sizes, 2 * n_hops);
    DGS_LAUNCH_CHECK();
    return DGS_OK;
  }
  DGS_REQUIRE(seeds != nullptr, DGS_ERR_INVALID, "dgs_sample_blocks: null seeds");
  DGS_REQUIRE(workspace != nullptr && workspace_bytes >= dgs_sample_blocks_workspace_bytes(hops, n_hops) &&
                  (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
              DGS_ERR_INVALID, "dgs_sample_blocks: workspace too small or not 16-byte aligned");
  for (int h = 0; h < n_hops; ++h) {
    DGS_REQUIRE(hops[h].coo_row != nullptr && hops[h].coo_col != nullptr && hops[h].frontier != nullptr,
                DGS_ERR_INVALID, "dgs_sample_blocks: hop %d: null output", h);
    DGS_REQUIRE(probs == nullptr || replace || hops[h].fanout <= 32, DGS_ERR_UNSUPPORTED,
                "dgs_sample_blocks: weighted fan-out %lld > 32 without replacement is not supported",
                (long long)hops[h].fanout);
  }

  // ---- carve the workspace ----
  char* p = static_cast<char*>(workspace);
  int64_t* n0_dev = reinterpret_cast<int64_t*>(p);
  p += WS_ALIGN;
  void* plan[DGS_MAX_HOPS];
  void* table[DGS_MAX_HOPS];
  static_assert(sizeof(int64_t) * (1 + DGS_MAX_HOPS) <= WS_ALIGN, "the control words hold n0 and one key per hop");
  uint64_t* keys_dev = reinterpret_cast<uint64_t*>(n0_dev + 1);
  InitWords init{n0_dev, n0, 0, {}, rng_words, keys_dev, n_hops};
  for (int h = 0; h < n_hops; ++h) {
    const int64_t key_bound = hops[h].seed_bound * (1 + hops[h].fanout);
    plan[h] = p;
    p += ws_align(dgs_sample_plan_bytes(hops[h].seed_bound));
    table[h] = p;
    p += ws_align(dgs_relabel_table_bytes(key_bound));
    init.tickets[init.n_tickets++] = sample_plan_ticket(plan[h], hops[h].seed_bound);
    init.tickets[init.n_tickets++] = unique_ticket(table[h], key_bound);
  }
  DGS_CUDA_TRY(launch_chained(SITE_INIT, blocks_init_kernel, 1u, 32u, s, init));

  // one-word table slots when every node id fits 32 bits (relabel_device.cuh); DGS_RELABEL_WIDE=1 keeps the
  // two-word slots for comparison
  static const bool force_wide = [] {
    const char* e = std::getenv("DGS_RELABEL_WIDE");
    return e != nullptr && e[0] == '1';
  }();
  const bool compact = !force_wide && (!ids64 || indptr->total - 1 < COMPACT_KEY_LIMIT);

  // ---- queue every hop; no size is read back in between ----
  const void* hop_seeds = seeds;
  const int64_t* n_dev = n0_dev;
  LookupJob pending{};  // relabelling of the previous hop's COO, carried by the next plan launch
  SizesReport report{};
  report.dst = sizes;
  for (int h = 0; h < n_hops; ++h) {
    const dgs_hop& hp = hops[h];
    const int64_t k = hp.fanout;
    const int64_t edge_bound = hp.seed_bound * k;
    const int64_t key_bound = hp.seed_bound + edge_bound;
    const Count n{hp.seed_bound, n_dev, nullptr};
    // the table is dimensioned before the neighbours are drawn: seeds * (1 + fanout) keys at most
    const TableSize size{n, 1 + k, compact};
    rc = launch_sample_plan(*indptr, hop_seeds, ids64 != 0, n, k, replace != 0, plan[h], nullptr, false,
                            make_clear_job(table[h], key_bound, size), pending, status, s);
    if (rc != DGS_OK) return rc;
    const int64_t* nnz_dev = sample_plan_total(plan[h], hp.seed_bound);
    const RngKey key = rng_words != nullptr
                           ? RngKey{0, keys_dev + h}
                           : host_key(sample_rng_key(rng_seed, rng_offset + static_cast<uint64_t>(h)));
    const bool row_is_position = h > 0;
    rc = probs != nullptr
             ? launch_sample_weighted(*indices, *probs, hop_seeds, ids64 != 0, n, k, replace != 0, plan[h],
                                      key, hp.coo_row, hp.coo_col, edge_bound, nullptr, row_is_position, status, s)
             : launch_sample_uniform(*indices, hop_seeds, ids64 != 0, n, k, replace != 0, plan[h], key,
                                     hp.coo_row, hp.coo_col, edge_bound, nullptr, row_is_position, status, s);
    if (rc != DGS_OK) return rc;
    const Count nnz{edge_bound, nnz_dev, nullptr};
    report.src[2 * h] = nnz_dev;
    report.src[2 * h + 1] = unique_total(table[h], key_bound);
    if (h == n_hops - 1) report.n = 2 * n_hops;  // the last hop's count kernel sends all sizes to the host at once
    rc = launch_unique_pair(ids64 != 0, hop_seeds, n, hp.coo_col, nnz, key_bound, size, table[h], hp.frontier,
                            hp.frontier_bound, nullptr, report, status, s);
    if (rc != DGS_OK) return rc;
    pending = make_lookup_job(table[h], key_bound, size, row_is_position ? nullptr : hp.coo_row, hp.coo_col, nnz,
                              hp.coo_row, hp.coo_col);
    hop_seeds = hp.frontier;
    n_dev = unique_total(table[h], key_bound);
  }
  return launch_lookup(pending, ids64 != 0, s);
}

}  // namespace
}  // namespace dgs

extern "C" int dgs_sample_blocks(const dgs_chunk_desc* indptr, const dgs_chunk_desc* indices,
                                 const dgs_chunk_desc* probs, const void* seeds, int32_t ids64,
                                 const dgs_hop* hops, int32_t n_hops, int32_t replace, uint64_t rng_seed,
                                 uint64_t rng_offset, void* workspace, size_t workspace_bytes,
                                 int64_t* sizes, int32_t* status, dgs_stream_t stream) {
  return dgs::queue_blocks(indptr, indices, probs, seeds, ids64, hops, n_hops, replace, rng_seed, rng_offset, nullptr,
                           workspace, workspace_bytes, sizes, status, stream);
}

// ---- the sequence recorded once and replayed ------------------------------------
// Queuing a batch is ~18 kernel launches with the same parameters every time as long as the buffers, the
// bounds (the number of seeds) and the tables stay the same; only the random stream differs.  A recording
// holds those launches as one executable graph (stream capture keeps the programmatic edges between the
// kernels), and a replay is a single launch call.
struct dgs_blocks_recording {
  cudaGraphExec_t exec = nullptr;
};

extern "C" int dgs_sample_blocks_record(const dgs_chunk_desc* indptr, const dgs_chunk_desc* indices,
                                        const dgs_chunk_desc* probs, const void* seeds, int32_t ids64,
                                        const dgs_hop* hops, int32_t n_hops, int32_t replace,
                                        const uint64_t* rng_words, void* workspace, size_t workspace_bytes,
                                        int64_t* sizes, int32_t* status, dgs_stream_t capture_stream,
                                        dgs_blocks_recording** out) {
  using namespace dgs;
  DGS_REQUIRE(out != nullptr && rng_words != nullptr, DGS_ERR_INVALID, "dgs_sample_blocks_record: null argument");
  DGS_REQUIRE(capture_stream != nullptr, DGS_ERR_INVALID,
              "dgs_sample_blocks_record: the default stream cannot record; pass a stream of your own");
  *out = nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(capture_stream);
  // thread-local mode: other host threads keep allocating and copying while this one records
  DGS_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  const int rc = queue_blocks(indptr, indices, probs, seeds, ids64, hops, n_hops, replace, 0, 0, rng_words, workspace,
                              workspace_bytes, sizes, status, capture_stream);
  cudaGraph_t graph = nullptr;
  const cudaError_t end = cudaStreamEndCapture(s, &graph);  // always closed, also after a refused argument
  if (rc != DGS_OK) {
    if (graph != nullptr) cudaGraphDestroy(graph);
    (void)cudaGetLastError();
    return rc;
  }
  if (end != cudaSuccess) return cuda_fail(end, "cudaStreamEndCapture", __FILE__, __LINE__);
  cudaGraphExec_t exec = nullptr;
  const cudaError_t inst = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (inst != cudaSuccess) return cuda_fail(inst, "cudaGraphInstantiate", __FILE__, __LINE__);
  dgs_blocks_recording* rec = new (std::nothrow) dgs_blocks_recording;
  if (rec == nullptr) {
    cudaGraphExecDestroy(exec);
    DGS_REQUIRE(false, DGS_ERR_CUDA, "dgs_sample_blocks_record: out of host memory");
  }
  rec->exec = exec;
  *out = rec;
  return DGS_OK;
}

extern "C" int dgs_sample_blocks_replay(dgs_blocks_recording* rec, dgs_stream_t stream) {
  using namespace dgs;
  DGS_REQUIRE(rec != nullptr && rec->exec != nullptr, DGS_ERR_INVALID, "dgs_sample_blocks_replay: null recording");
  DGS_CUDA_TRY(cudaGraphLaunch(rec->exec, static_cast<cudaStream_t>(stream)));
  return DGS_OK;
}

extern "C" void dgs_sample_blocks_recording_free(dgs_blocks_recording* rec) {
  if (rec == nullptr) return;
  if (rec->exec != nullptr) cudaGraphExecDestroy(rec->exec);
  delete rec;
}
