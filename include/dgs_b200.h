/*
 * dgs_b200.h -- C ABI of the B200-native Dist-GPU-sampling hot path.
 *
 * Everything a foreign-function binding needs: plain pointers, sizes and POD
 * structs, `extern "C"` linkage, no torch / C++ types.  The PyTorch
 * custom-class library (libdgs.so) is a thin host layer on top of this file;
 * any other host (ctypes, cgo, JNI ...) can bind the same symbols.
 *
 * Conventions
 *   - every function returns DGS_OK (0) or a DGS_ERR_* code; the text of the
 *     last failure on the calling thread is returned by dgs_last_error().
 *   - kernels are enqueued on the `stream` argument (a cudaStream_t passed as
 *     void*; NULL = legacy default stream, which is what the reference uses)
 *     and the call returns without synchronising unless stated otherwise.
 *   - no function allocates device memory except dgs_store_create /
 *     dgs_comm_init; outputs and scratch are passed in by the caller.
 *   - "ids" (seeds, row ids, indptr, indices) are int64 when `ids64 != 0`,
 *     int32 otherwise -- the two id types the reference dispatches
 *     (src/dgs_headers.h:47-59 DGS_ID_TYPE_SWITCH).
 *   - data-dependent sizes (nnz, number of unique keys, split counts) are
 *     written by the kernels through a pointer that must be device-writable;
 *     pass pinned (cudaHostAlloc) memory and read it after synchronising the
 *     stream.
 *
 * Each entry point names the reference interface it replaces
 * (path:line inside gpzlx1/Dist-GPU-sampling).
 */
#ifndef DGS_B200_H_
#define DGS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DGS_API __attribute__((visibility("default")))
#else
#define DGS_API
#endif

#define DGS_MAX_PARTS 8

enum {
  DGS_OK = 0,
  DGS_ERR_INVALID = 1,     /* bad argument */
  DGS_ERR_CUDA = 2,        /* a CUDA runtime call failed */
  DGS_ERR_NCCL = 3,        /* an NCCL call failed */
  DGS_ERR_SHM = 4,         /* shared-memory host tail could not be set up */
  DGS_ERR_UNSUPPORTED = 5, /* size / dtype outside what the kernels handle */
  DGS_ERR_RANGE = 6,       /* a kernel met an out-of-range id (status word) */
  DGS_ERR_TABLE_FULL = 7,  /* hash table probe ran out of slots (status word) */
  DGS_ERR_MISMATCH = 8     /* ranks disagree on the ChunkTensor metadata */
};

typedef void* dgs_stream_t; /* cudaStream_t */

/*
 * Placement of one ChunkTensor, passed BY VALUE to every kernel.
 * Replaces the device-resident `chunk_tensor_wrapper<T>` (src/chunk_tensor.h:10-59):
 * flat element e lives
 *   - on GPU p = e / each at element offset e - p*each      if e <  threshold
 *   - in the host tail at element offset e - threshold       if e >= threshold
 * A plain (non-chunked) device tensor is the special case num_parts = 1,
 * threshold = each = total, dev[0] = data pointer.
 */
typedef struct dgs_chunk_desc {
  int64_t total;      /* number of elements of the whole tensor            */
  int64_t threshold;  /* elements resident on GPUs: each * num_parts, clamped */
  int64_t each;       /* elements per GPU chunk                            */
  int32_t num_parts;  /* GPUs sharing the tensor (1..DGS_MAX_PARTS)        */
  int32_t local_rank; /* this process' chunk                               */
  int32_t esz;        /* element size in bytes (1, 2, 4 or 8)              */
  int32_t reserved;
  const void* host;   /* device-visible base of the host tail, or NULL     */
  const void* dev[DGS_MAX_PARTS]; /* device-visible base of every chunk   */
} dgs_chunk_desc;

DGS_API const char* dgs_last_error(void);
/* sm_100a fatbin check + device properties; DGS_ERR_CUDA when no usable GPU. */
DGS_API int dgs_device_check(void);

/* ---- placement arithmetic (pure host code, no CUDA) -------------------- */
/* ChunkTensor::ChunkTensor size rules, src/chunk_tensor.cc:53-73. */
DGS_API int dgs_placement(int64_t total_elems, int32_t esz, int64_t capacity_per_gpu_bytes,
                  int32_t world, int64_t* each, int64_t* threshold,
                  int64_t* host_elems);

/* ---- communicator (bootstrap only) ------------------------------------- */
/* nccl::GetUniqueId, src/nccl_context.cc:17-22: 128-byte id as int64[16]. */
DGS_API int dgs_comm_get_unique_id(int64_t* id16);
/* nccl::SetNCCL, src/nccl_context.cc:24-34. */
DGS_API int dgs_comm_init(int64_t nranks, const int64_t* id16, int64_t rank);
/* nccl::_Barrier, src/nccl_context.cc:36-40. */
DGS_API int dgs_comm_barrier(void);
DGS_API int dgs_comm_rank(void);  /* 0 when no communicator was set */
DGS_API int dgs_comm_size(void);  /* 1 when no communicator was set */
DGS_API int dgs_comm_destroy(void);

/* ---- HMGStore: one ChunkTensor's memory -------------------------------- */
typedef struct dgs_store dgs_store;

/* ChunkTensor::ChunkTensor, src/chunk_tensor.cc:37-149.  Collective over the
 * communicator.  `shape` has 1 or 2 dims; `esz` is the element size. */
DGS_API int dgs_store_create(const int64_t* shape, int32_t ndim, int32_t esz,
                     int64_t capacity_per_gpu_bytes, dgs_store** out);
/* ChunkTensor::_Free, src/chunk_tensor.cc:235-263.  Collective. */
DGS_API int dgs_store_destroy(dgs_store* s);
/* The by-value accessor that replaces wrapper_chunktensor_ptr_
 * (src/chunk_tensor.cc:223-233). */
DGS_API int dgs_store_desc(const dgs_store* s, dgs_chunk_desc* out);
/* row width: strides_[0] (src/chunk_tensor.cc:46-52). */
DGS_API int64_t dgs_store_elem_stride(const dgs_store* s);
/* ChunkTensor::LoadFromTensor, src/chunk_tensor.cc:173-200: called on ONE
 * rank with the whole contiguous host tensor; synchronous. */
DGS_API int dgs_store_load(dgs_store* s, const void* host_data, int64_t n_elems);
/* ChunkTensor::GetHostTensor / GetSubDeviceTensor, src/chunk_tensor.cc:151-171:
 * flat views; *ptr = NULL and *n_elems = 0 when that part is empty. */
DGS_API int dgs_store_host_view(const dgs_store* s, void** ptr, int64_t* n_elems);
DGS_API int dgs_store_local_view(const dgs_store* s, void** ptr, int64_t* n_elems);
/* CUDAContext::GetCurrAllocated, src/cuda_context.h:11-38. */
DGS_API int64_t dgs_alloc_current_bytes(void);

/* ---- sticky device status ---------------------------------------------- */
/* Kernels never trap: an out-of-range id or a full hash table sets a status
 * word (replaces the device asserts of src/cuda/*.cu).  `status` arguments
 * below are device-writable int32 words (pinned memory is fine) or NULL. */

/* ---- row gather -------------------------------------------------------- */
enum { DGS_CLASS_ANY = 0, DGS_CLASS_LOCAL = 1, DGS_CLASS_REMOTE = 2, DGS_CLASS_HOST = 3 };
/* IndexFromChunkTensorCUDA / Local.. / Remote.. / Host..,
 * src/cuda/index_with_chunk_tensor.cu:29-53,170-247:
 *   out[i*D + j] = T.At(idx[i]*D + j),  i < n, j < D.
 * `location_class` is a hint only (all classes resolve the owner per row, so
 * the result is the same for ids of any class).  A row id outside the tensor
 * yields a zero row and DGS_ERR_RANGE in *status. */
DGS_API int dgs_gather_rows(const dgs_chunk_desc* t, int32_t location_class,
                    const void* idx, int32_t ids64, int64_t n, int64_t D,
                    void* out, int32_t* status, dgs_stream_t stream);

/* dgs_gather_rows for a request whose length is only known on the device: the
 * kernel gathers min(*n_dev, n_bound) rows, n_dev being a device word that an
 * earlier kernel on the same stream writes (e.g. the frontier length of
 * dgs_sample_blocks, see dgs_sample_blocks_frontier_count); the host sizes
 * `out` for n_bound rows.  This lets the feature gather of a mini-batch
 * (features._CAPI_index(input_nodes) in the reference's training loop,
 * oppo_bench/single_node/chunktensor.py:147-150) be queued directly behind the
 * sampling sequence, without the host reading the frontier length first.
 * No counterpart in the reference, which reads every size back. */
DGS_API int dgs_gather_rows_counted(const dgs_chunk_desc* t, const void* idx, int32_t ids64,
                                    int64_t n_bound, const int64_t* n_dev, int64_t D,
                                    void* out, int32_t* status, dgs_stream_t stream);

/* SplitIndexFromChunkTensorCUDA, src/cuda/index_with_chunk_tensor.cu:55-108.
 * Stable 3-way partition of the ids: out = [local ids | remote ids | host ids]
 * (each class in input order), counts[0..2] = class sizes.  */
DGS_API size_t dgs_split_index_scratch_bytes(int64_t n);
DGS_API int dgs_split_index(const dgs_chunk_desc* t, const void* idx, int32_t ids64,
                    int64_t n, int64_t D, void* out, int64_t* counts,
                    void* scratch, size_t scratch_bytes, dgs_stream_t stream);

/* Same result as dgs_split_index, for hosts that must not allocate: the three
 * kernels keep their tile counters in a 192 KB array that is part of the
 * library image instead of caller scratch, and the call itself performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.  It is meant
 * for callers that receive all their buffers up front and then run with the
 * allocator off limits -- a plug-in inside a serving process with a fixed
 * memory budget, or a latency-critical loop that cannot afford the
 * device-wide synchronisation cudaMalloc and cudaFree may cause.  `out` and
 * `counts` are still supplied by the caller.
 * Limits and rules:
 *   - at most DGS_SPLIT_STATIC_MAX_IDS ids per call; larger n is rejected with
 *     DGS_ERR_UNSUPPORTED before anything is launched;
 *   - the first call on each device looks up the array's device address (with
 *     that device current); make that first call before any stream capture;
 *   - all calls on one device share the one array, which keeps whatever the
 *     previous call left in it: calls whose kernels can overlap on the GPU
 *     (different streams without ordering between them) race and must be
 *     serialised by the caller.  Nothing has to be cleared between calls:
 *     every word a call reads it has written itself.
 * This entry point has no counterpart in the reference. */
#define DGS_SPLIT_STATIC_MAX_IDS (1 << 24)
DGS_API int dgs_split_index_static(const dgs_chunk_desc* t, const void* idx, int32_t ids64,
                                   int64_t n, int64_t D, void* out, int64_t* counts,
                                   dgs_stream_t stream);

/* ---- row-wise neighbour sampling --------------------------------------- */
/* Plan = per-seed row range and output offsets.
 * _GetSubIndptr + cub_exclusiveSum, src/cuda/rowwise_sampling.cu:13-40 and the
 * row_begin/row_end pre-gather of
 * src/cuda/rowwise_sampling_with_chunk_tensor.cu:136-153.
 * count(seed) = min(deg,k) without replacement, (deg ? k : 0) with.
 * `plan` is caller scratch of dgs_sample_plan_bytes(n) bytes that must stay
 * alive until the matching dgs_sample_* call has run.  If nnz != NULL the
 * total output size is written there by the plan kernel itself (its last CTA),
 * i.e. before any sampling kernel enqueued behind it has run. */
DGS_API size_t dgs_sample_plan_bytes(int64_t n_seeds);
DGS_API int dgs_sample_plan(const dgs_chunk_desc* indptr, const void* seeds, int32_t ids64,
                    int64_t n_seeds, int64_t k, int32_t replace, void* plan,
                    int64_t* nnz, int32_t* status, dgs_stream_t stream);

/* RowWiseSamplingUniformCUDA / ...WithChunkTensorCUDA,
 * src/cuda/rowwise_sampling.cu:138-187,
 * src/cuda/rowwise_sampling_with_chunk_tensor.cu:113-194.
 * COO output grouped by seed position; rows with deg <= k (no replacement)
 * are copied whole in CSC order; other rows get k uniform picks (distinct
 * positions unless `replace`).  coo_row/coo_col hold out_capacity ids
 * (n_seeds*k always suffices).  If nnz != NULL the total is written there.
 * If picked_pos != NULL it receives, per output, the position inside the row
 * (int64) -- a test hook for multigraph validity checks.
 * Randomness: Philox4x32-10 keyed by `rng_seed`, counter from `rng_offset`
 * and the seed position; identical arguments give identical output. */
DGS_API int dgs_sample_uniform(const dgs_chunk_desc* indices, const void* seeds,
                       int32_t ids64, int64_t n_seeds, int64_t k, int32_t replace,
                       const void* plan, uint64_t rng_seed, uint64_t rng_offset,
                       void* coo_row, void* coo_col, int64_t out_capacity,
                       int64_t* nnz, int64_t* picked_pos, int32_t* status,
                       dgs_stream_t stream);

/* RowWiseSamplingProbCUDA / ...WithChunkTensorCUDA,
 * src/cuda/rowwise_sampling_probs.cu:218-282,
 * src/cuda/rowwise_sampling_probs_with_chunk_tensor.cu:180-296.
 * `probs` holds one fp32 weight per edge.  Without replacement: A-Res
 * (keep the k largest u^(1/w)); k <= 32 as in the reference (:65).
 * With replacement: k draws proportional to max(w,0). */
DGS_API int dgs_sample_weighted(const dgs_chunk_desc* indices, const dgs_chunk_desc* probs,
                        const void* seeds, int32_t ids64, int64_t n_seeds,
                        int64_t k, int32_t replace, const void* plan,
                        uint64_t rng_seed, uint64_t rng_offset, void* coo_row,
                        void* coo_col, int64_t out_capacity, int64_t* nnz,
                        int64_t* picked_pos, int32_t* status, dgs_stream_t stream);

/* ---- unique / relabel --------------------------------------------------- */
#define DGS_MAX_SEGMENTS 8
/* A logical concatenation of up to DGS_MAX_SEGMENTS device arrays (replaces
 * the torch::cat calls of src/cuda/tensor_reindex.cu:190,197). */
typedef struct dgs_segments {
  int32_t count;
  int32_t reserved;
  const void* ptr[DGS_MAX_SEGMENTS];
  int64_t len[DGS_MAX_SEGMENTS];
} dgs_segments;

/* Unique, src/cuda/tensor_reindex.cu:82-159 (+ RelabelHashmap :11-75).
 * unique_out (capacity = total key count) receives the distinct keys in
 * first-occurrence order; *n_unique their number.  `table` is caller scratch
 * of dgs_relabel_table_bytes(total keys) bytes and afterwards maps
 * key -> position in unique_out for dgs_relabel_lookup.  Keys must be >= 0
 * (negative keys are skipped and reported as DGS_ERR_RANGE). */
DGS_API size_t dgs_relabel_table_bytes(int64_t n_keys);
DGS_API int dgs_unique_first_occurrence(const dgs_segments* keys, int32_t ids64,
                                void* table, size_t table_bytes, void* unique_out,
                                int64_t* n_unique, int32_t* status,
                                dgs_stream_t stream);
/* Relabel, src/cuda/tensor_reindex.cu:161-180: out = position of each input id
 * in unique_out, or -1 when absent.  `out` is one contiguous array holding the
 * segments back to back. */
DGS_API int dgs_relabel_lookup(const void* table, size_t table_bytes, int64_t n_keys_built,
                       const dgs_segments* in, int32_t ids64, void* out,
                       dgs_stream_t stream);

/* ---- multi-hop sample + relabel, queued as one sequence ---------------- */
/* Replaces the hop loop of ChunkTensorSampler.sample_blocks (reference
 * oppo_bench/single_node/utils/chunktensor_sampler.py:93-118): for every fan-out,
 * last one first as there, sample the current seeds, take the first-occurrence
 * unique list of (seeds ++ sampled neighbours) as the next hop's seeds, and
 * relabel the hop's COO into positions of that list -- what the reference does
 * with one _CAPI_sample_neighbors* and one _CAPI_tensor_relabel call per hop,
 * each with a blocking size read-back.  Here no size is read back while the
 * sequence runs: buffers are sized by upper bounds (dgs_sample_blocks_bounds),
 * every kernel takes its item count from a device word written by the kernel
 * before it, and the actual sizes are written to `sizes` for one read at the end.
 *
 * hops[] is in the order of APPLICATION (hops[0] samples the caller's seeds).
 * On return (after the stream reaches this point), for hop h:
 *   sizes[2h]   = nnz_h: valid entries of coo_row / coo_col
 *   sizes[2h+1] = valid entries of frontier (= number of seeds of hop h+1)
 *   coo_row[e]  = index in frontier_h of the seed that edge e was sampled for
 *                 (the seeds come first in frontier_h, in order, so for a
 *                 duplicate-free seed list this is the seed's position)
 *   coo_col[e]  = index of the sampled neighbour in frontier_h
 * Results are the same as the per-hop operators give (same grouping by seed,
 * whole rows in CSC order, first-occurrence numbering); stochastic rows use the
 * random stream (rng_seed, rng_offset + h). */
#define DGS_MAX_HOPS 8
typedef struct dgs_hop {
  int64_t fanout;
  int64_t seed_bound;     /* capacity of this hop's seed list; hop 0: the exact number of seeds */
  int64_t frontier_bound; /* capacity of `frontier`; equals seed_bound of the next hop */
  void* coo_row;          /* [seed_bound * fanout] ids */
  void* coo_col;          /* [seed_bound * fanout] ids */
  void* frontier;         /* [frontier_bound] ids */
} dgs_hop;

/* Fills fanout / seed_bound / frontier_bound of hops[0..n_hops): hop h can reach
 * at most seed_bound * (1 + fanout) distinct nodes and never more than num_nodes. */
DGS_API int dgs_sample_blocks_bounds(int64_t n_seeds, const int64_t* fanouts, int32_t n_hops,
                                     int64_t num_nodes, dgs_hop* hops);
DGS_API size_t dgs_sample_blocks_workspace_bytes(const dgs_hop* hops, int32_t n_hops);
/* probs == NULL: uniform sampling.  workspace: device memory, 16-byte aligned,
 * contents irrelevant.  sizes: [2 * n_hops] int64, device-writable (pinned). */
DGS_API int dgs_sample_blocks(const dgs_chunk_desc* indptr, const dgs_chunk_desc* indices,
                              const dgs_chunk_desc* probs, const void* seeds, int32_t ids64,
                              const dgs_hop* hops, int32_t n_hops, int32_t replace,
                              uint64_t rng_seed, uint64_t rng_offset, void* workspace,
                              size_t workspace_bytes, int64_t* sizes, int32_t* status,
                              dgs_stream_t stream);

/* Device address (inside `workspace`) of the word that holds the length of the
 * last hop's frontier once the sequence queued by dgs_sample_blocks with the same
 * hops / workspace has run: the n_dev of dgs_gather_rows_counted.  NULL on bad
 * arguments.  No counterpart in the reference. */
DGS_API const int64_t* dgs_sample_blocks_frontier_count(const dgs_hop* hops, int32_t n_hops,
                                                        void* workspace);

/* The same sequence recorded once and replayed: queuing a batch through
 * dgs_sample_blocks costs about eighteen kernel launches whose parameters do not
 * change while buffers, bounds (hence the number of seeds) and graph stay the same.
 * dgs_sample_blocks_record captures them on `capture_stream` (a stream of the
 * caller's own, not the default stream; nothing runs) into one executable graph;
 * dgs_sample_blocks_replay queues that graph on a stream with a single call.
 * What differs between replays comes from memory: the seeds (rewrite the `seeds`
 * buffer) and the random stream, read by the first kernel of every replay from
 * rng_words[0] (seed) and rng_words[1] (offset) -- device-readable memory the host
 * can write, i.e. pinned; hop h uses (seed, offset + h) like dgs_sample_blocks, so
 * a replay gives bit for bit what dgs_sample_blocks gives for the same words.
 * One replay of a recording at a time (they share the workspace and outputs).
 * The arguments are those of dgs_sample_blocks.  No counterpart in the reference. */
typedef struct dgs_blocks_recording dgs_blocks_recording;
DGS_API int dgs_sample_blocks_record(const dgs_chunk_desc* indptr, const dgs_chunk_desc* indices,
                                     const dgs_chunk_desc* probs, const void* seeds, int32_t ids64,
                                     const dgs_hop* hops, int32_t n_hops, int32_t replace,
                                     const uint64_t* rng_words, void* workspace,
                                     size_t workspace_bytes, int64_t* sizes, int32_t* status,
                                     dgs_stream_t capture_stream, dgs_blocks_recording** out);
DGS_API int dgs_sample_blocks_replay(dgs_blocks_recording* rec, dgs_stream_t stream);
DGS_API void dgs_sample_blocks_recording_free(dgs_blocks_recording* rec);

/* ---- PaGraph-style feature cache ---------------------------------------- */
/* CreateHashMapTensorCUDA, src/cuda/pagraph.cu:94-124: open-addressing table
 * key -> value with capacity dgs_cache_table_slots(n); key_buf/value_buf hold
 * that many ids (empty key = -1). */
DGS_API int64_t dgs_cache_table_slots(int64_t n_keys);
DGS_API int dgs_cache_build(const void* keys, const void* values, int32_t ids64,
                    int64_t n_keys, void* key_buf, void* value_buf,
                    int64_t slots, int32_t* status, dgs_stream_t stream);
/* FetchDataCUDA / FetchDataWithChunkTensorCUDA, src/cuda/pagraph.cu:196-262:
 * row nid[i] comes from the GPU cache (row value of the table, read through
 * `gpu_data`) on a hit, else from the device-visible host array
 * `cpu_data[nid[i]*D ...]` of cpu_rows rows (ids beyond it give a zero row
 * and DGS_ERR_RANGE). */
DGS_API int dgs_cache_fetch(const void* cpu_data, int64_t cpu_rows, const dgs_chunk_desc* gpu_data,
                    const void* nid, int32_t ids64, int64_t n, int64_t D,
                    const void* key_buf, const void* value_buf, int64_t slots,
                    void* out, int32_t* status, dgs_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* DGS_B200_H_ */
