// Internal launchers shared between the per-operator entry points (sample.cu,
// relabel.cu) and the multi-hop sequence (blocks.cu).  Not part of the C ABI.
#pragma once
#include "common.cuh"
#include "relabel_device.cuh"

namespace dgs {

// ---- sample.cu ---------------------------------------------------------------
// `plan` is laid out for n.bound seeds.  nnz_out (optional, normally pinned)
// receives the number of sampled edges; the same number stays in the plan at
// sample_plan_total().  The plan's ticket word must be zero at launch: it is
// cleared here when zero_ticket is set and resets itself after every use.
// clear / lookup (either may have ctas == 0): independent jobs run by extra CTAs of
// the plan launch -- clearing the table this hop will fill, relabelling the COO of
// the hop before it.
int launch_sample_plan(const dgs_chunk_desc& indptr, const void* seeds, bool ids64, Count n, int64_t k,
                       bool replace, void* plan, int64_t* nnz_out, bool zero_ticket, const ClearJob& clear,
                       const LookupJob& lookup, int32_t* status, cudaStream_t s);
int64_t* sample_plan_total(void* plan, int64_t n_bound);
unsigned int* sample_plan_ticket(void* plan, int64_t n_bound);

// row_is_position: write the seed's position in the seed list to coo_row instead
// of the seed id (valid as a relabelled id when the seed list has no duplicates).
int launch_sample_uniform(const dgs_chunk_desc& indices, const void* seeds, bool ids64, Count n, int64_t k,
                          bool replace, void* plan, RngKey key, void* coo_row,
                          void* coo_col, int64_t out_capacity, int64_t* picked_pos, bool row_is_position,
                          int32_t* status, cudaStream_t s);
int launch_sample_weighted(const dgs_chunk_desc& indices, const dgs_chunk_desc& probs, const void* seeds,
                           bool ids64, Count n, int64_t k, bool replace, void* plan,
                           RngKey key, void* coo_row, void* coo_col, int64_t out_capacity,
                           int64_t* picked_pos, bool row_is_position, int32_t* status, cudaStream_t s);
uint64_t sample_rng_key(uint64_t rng_seed, uint64_t rng_offset);

// ---- relabel.cu ----------------------------------------------------------------
// `table` is laid out for key_bound keys (dgs_relabel_table_bytes(key_bound)); `size`
// says how much of it is in use (cleared, probed); every kernel of one table gets
// the same TableSize.
ClearJob make_clear_job(void* table, int64_t key_bound, const TableSize& size);
LookupJob make_lookup_job(const void* table, int64_t key_bound, const TableSize& size, const void* a, const void* b,
                          Count n, void* out_a, void* out_b);
int launch_clear(const ClearJob& job, cudaStream_t s);            // as a launch of its own
int launch_lookup(const LookupJob& job, bool ids64, cudaStream_t s);

// First-occurrence unique of the logical concatenation a[0:na) ++ b[0:nb) whose
// lengths are device words, into a table that has been cleared.  unique_out holds
// unique_capacity ids; a larger result raises DGS_ERR_RANGE in the status word and
// is cut off.  The table's ticket word must be zero at launch (it resets itself).  `report`
// (n may be 0) is carried out by the kernel that knows the number of distinct keys.
int launch_unique_pair(bool ids64, const void* a, Count na, const void* b, Count nb, int64_t key_bound,
                       const TableSize& size, void* table, void* unique_out, int64_t unique_capacity,
                       int64_t* n_unique_out, const SizesReport& report, int32_t* status, cudaStream_t s);
int64_t* unique_total(void* table, int64_t key_bound);
unsigned int* unique_ticket(void* table, int64_t key_bound);

}  // namespace dgs
