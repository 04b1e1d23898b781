// Unique (first-occurrence order) + relabel through an open-addressing table.
//
// Replaces RelabelHashmap / Unique / Relabel / TensorRelabelCUDA
// (reference src/cuda/tensor_reindex.cu:11-205): three torch::full tables, two
// torch::cat copies, four thrust passes that each re-probe the table, a cub
// scan and a blocking read-back, with hash(key) = key & (cap-1) at a load
// factor of up to 100 %.
//
// Kept (the contract): the i-th distinct key in first-occurrence order gets
// label i; lookups return the label or -1.  The order is fixed by storing the
// MINIMUM input index per key (atomicMin) exactly as the reference does
// (:28,123), so the result does not depend on hash layout or thread timing.
//
// Different (the design):
//   * one 16-byte slot {key, value} per entry (a probe touches one sector, not
//     three arrays), mixed 64-bit hash, linear probing, load factor <= 50 %.
//   * inputs are read through a segment list instead of being concatenated.
//   * the insert pass remembers each input's slot, so later passes index the
//     table directly instead of probing again.
//   * numbering is count-per-tile (the last CTA to finish scans the tile sums,
//     no extra launch) -> write; the label is
//     stored into the slot's value with the top bit set, which can never be
//     mistaken for an input index by a concurrent reader, so no third table.
//   * the number of distinct keys goes to a caller-supplied (pinned) word.
#include "common.cuh"
#include "launchers.h"
#include "relabel_device.cuh"
#include "philox.cuh"
#include "tile_scan.cuh"

namespace dgs {
namespace {

constexpr int RL_ITEMS = 4;
constexpr int RL_TILE = RL_BLOCK * RL_ITEMS;

struct TableView {
  Slot* slots;         // [cap]
  uint32_t* slot_of;   // [n]  slot of every input
  int64_t* tile_off;   // [ntiles]
  int64_t* total;      // [1]
  unsigned int* ticket;  // [1]
  uint64_t cap;
  int64_t ntiles;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline TableView table_view(void* mem, int64_t n) {
  TableView t;
  t.cap = slots_for(n);
  t.ntiles = (n + RL_TILE - 1) / RL_TILE;
  char* p = static_cast<char*>(mem);
  t.slots = reinterpret_cast<Slot*>(p);
  p += t.cap * sizeof(Slot);
  t.slot_of = reinterpret_cast<uint32_t*>(p);
  p += align_up(static_cast<size_t>(n) * sizeof(uint32_t), 16);
  t.tile_off = reinterpret_cast<int64_t*>(p);
  t.total = t.tile_off + t.ntiles;
  t.ticket = reinterpret_cast<unsigned int*>(t.total + 1);
  return t;
}

// ---- where the keys come from ---------------------------------------------------
// A host-known segment list (the per-operator entry points) ...
struct SegKeys {
  dgs_segments s;
  int64_t n;
  __device__ __forceinline__ int64_t size() const { return n; }
  __device__ __forceinline__ int64_t bound() const { return n; }
  template <typename IdT>
  __device__ __forceinline__ IdT load(int64_t i) const {
    return seg_load<IdT>(s, i);
  }
};
// ... or two arrays a[0:na) ++ b[0:nb) whose lengths are device words (the
// multi-hop sequence: a = this hop's seeds, b = the neighbours just sampled).
struct PairKeys {
  const void* a;
  const void* b;
  Count na, nb;
  __device__ __forceinline__ int64_t size() const { return count_of(na) + count_of(nb); }
  __device__ __forceinline__ int64_t bound() const { return na.bound + nb.bound; }
  template <typename IdT>
  __device__ __forceinline__ IdT load(int64_t i) const {
    const int64_t x = count_of(na);
    return i < x ? static_cast<const IdT*>(a)[i] : static_cast<const IdT*>(b)[i - x];
  }
};

// pass 0 of the sequence with device-side counts, when it does not ride on another
// launch: clear only the slots the table will use (the per-operator path clears
// with a memset instead)
__global__ void __launch_bounds__(RL_BLOCK) relabel_clear_kernel(const ClearJob job) {
  pdl_enter();
  run_clear_cta(job, blockIdx.x);
}

// pass 1: insert every key, keep the smallest input index per key
template <typename IdT, typename Keys>
__global__ void __launch_bounds__(RL_BLOCK)
relabel_insert_kernel(const __grid_constant__ Keys keys, const TableSize size, Slot* slots,
                      uint32_t* __restrict__ slot_of, int32_t* __restrict__ status) {
  pdl_enter();
  const int64_t n = keys.size();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * RL_BLOCK + threadIdx.x;
  if (i >= n) return;
  const uint64_t mask = table_slots(size) - 1;
  const long long key = static_cast<long long>(keys.template load<IdT>(i));
  if (key < 0 || (size.compact && key >= COMPACT_KEY_LIMIT)) {
    raise_status(status, DGS_ERR_RANGE);
    slot_of[i] = NO_SLOT;
    return;
  }
  uint32_t found = NO_SLOT;
  if (size.compact) {
    unsigned long long* words = reinterpret_cast<unsigned long long*>(slots);
    const uint32_t mask32 = static_cast<uint32_t>(mask), key32 = static_cast<uint32_t>(key);
    const unsigned long long mine = (static_cast<unsigned long long>(key32) << 32) | static_cast<unsigned long long>(i);
    uint32_t h = hash_key32(key32) & mask32;
    for (uint32_t probes = 0; probes <= mask32; ++probes) {
      unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(&words[h]);
      if (cur == EMPTY_COMPACT) {
        cur = atomicCAS(&words[h], EMPTY_COMPACT, mine);
        if (cur == EMPTY_COMPACT) {  // claimed, and the first index is in place: nothing else to do
          found = h;
          break;
        }
      }
      if (static_cast<uint32_t>(cur >> 32) == key32) {
        found = h;
        // same high half, so the minimum of the words is the minimum of the indices; a stale read can only
        // cause a redundant atomic (indices only ever decrease)
        if (static_cast<uint32_t>(cur) > static_cast<uint32_t>(i)) atomicMin(&words[h], mine);
        break;
      }
      h = (h + 1) & mask32;
    }
    slot_of[i] = found;
    if (found == NO_SLOT) raise_status(status, DGS_ERR_TABLE_FULL);
    return;
  }
  uint64_t h = hash_key(key) & mask;
  for (uint64_t probes = 0; probes <= mask; ++probes) {
    long long cur = *reinterpret_cast<volatile long long*>(&slots[h].key);
    if (cur == EMPTY_KEY)
      cur = static_cast<long long>(atomicCAS(reinterpret_cast<unsigned long long*>(&slots[h].key),
                                             static_cast<unsigned long long>(EMPTY_KEY),
                                             static_cast<unsigned long long>(key)));
    if (cur == EMPTY_KEY || cur == key) {
      found = static_cast<uint32_t>(h);
      break;
    }
    h = (h + 1) & mask;
  }
  slot_of[i] = found;
  if (found == NO_SLOT) {
    raise_status(status, DGS_ERR_TABLE_FULL);
    return;
  }
  // values only ever decrease, so a stale read can only cause a redundant atomic
  if (*reinterpret_cast<volatile unsigned long long*>(&slots[found].val) > static_cast<unsigned long long>(i))
    atomicMin(&slots[found].val, static_cast<unsigned long long>(i));
}

// pass 2: input i is a first occurrence iff the stored minimum equals i;
// the last CTA to finish turns the per-tile counts into offsets and publishes
// the number of distinct keys
__global__ void __launch_bounds__(RL_BLOCK)
relabel_count_kernel(const Count nc, const Slot* __restrict__ slots, const bool compact,
                     const uint32_t* __restrict__ slot_of, int64_t* tile_sums, unsigned int* ticket,
                     int64_t* total_dev, int64_t* n_unique_out, const SizesReport report) {
  __shared__ int s_cnt;
  __shared__ int64_t s_scan[RL_BLOCK / 32 + 1];
  pdl_enter();
  if (threadIdx.x == 0) s_cnt = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * RL_TILE + threadIdx.x * RL_ITEMS;
  // slot_of has room for nc.bound entries: read it while the live count is still on its way
  uint32_t sl[RL_ITEMS];
#pragma unroll
  for (int u = 0; u < RL_ITEMS; ++u) sl[u] = base + u < nc.bound ? slot_of[base + u] : NO_SLOT;
  const int64_t n = count_of(nc);
  int c = 0;
#pragma unroll
  for (int u = 0; u < RL_ITEMS; ++u) {
    const int64_t i = base + u;
    if (i < n && sl[u] != NO_SLOT) {
      const bool first =
          compact ? reinterpret_cast<const uint2*>(slots)[sl[u]].x == static_cast<uint32_t>(i)  // low half of the word
                  : slots[sl[u]].val == static_cast<unsigned long long>(i);
      if (first) ++c;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(FULL_MASK, c, o);
  if ((threadIdx.x & 31) == 0 && c) atomicAdd(&s_cnt, c);
  __syncthreads();
  const bool last = publish_and_scan_tiles<RL_BLOCK>(static_cast<int64_t>(s_cnt), tile_sums, ticket, total_dev,
                                                     n_unique_out, s_scan);
  if (last && threadIdx.x == 0 && report.n > 0) {  // same thread that wrote *total_dev just above
    for (int k = 0; k < report.n; ++k) report.dst[k] = *report.src[k];
    __threadfence_system();
  }
}

// pass 3: number the first occurrences, emit them, store the label in the slot
template <typename IdT, typename Keys>
__global__ void __launch_bounds__(RL_BLOCK)
relabel_number_kernel(const __grid_constant__ Keys keys, Slot* slots, const bool compact,
                      const uint32_t* __restrict__ slot_of,
                      const int64_t* __restrict__ tile_off, IdT* __restrict__ unique_out,
                      const int64_t unique_capacity, int32_t* __restrict__ status) {
  __shared__ int smem[RL_BLOCK / 32 + 1];
  pdl_enter();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * RL_TILE + threadIdx.x * RL_ITEMS;
  bool first[RL_ITEMS];
  uint32_t slot[RL_ITEMS];
  const int64_t room = keys.bound();
#pragma unroll
  for (int u = 0; u < RL_ITEMS; ++u) slot[u] = base + u < room ? slot_of[base + u] : NO_SLOT;  // ahead of the count
  const int64_t n = keys.size();
  int c = 0;
#pragma unroll
  for (int u = 0; u < RL_ITEMS; ++u) {
    const int64_t i = base + u;
    first[u] = false;
    if (i >= n) slot[u] = NO_SLOT;
    if (i < n) {
      // a slot already relabelled by another CTA carries LABEL_BIT and cannot equal i
      if (slot[u] != NO_SLOT)
        first[u] = compact ? *reinterpret_cast<const volatile uint32_t*>(reinterpret_cast<const uint2*>(slots) + slot[u]) ==
                                 static_cast<uint32_t>(i)
                           : *reinterpret_cast<const volatile unsigned long long*>(&slots[slot[u]].val) ==
                                 static_cast<unsigned long long>(i);
      c += first[u] ? 1 : 0;
    }
  }
  int total;
  const int ex = block_exclusive_scan<int, RL_BLOCK>(c, smem, &total);
  int64_t label = tile_off[blockIdx.x] + ex;
#pragma unroll
  for (int u = 0; u < RL_ITEMS; ++u) {
    if (first[u]) {
      if (label < unique_capacity) unique_out[label] = keys.template load<IdT>(base + u);
      else raise_status(status, DGS_ERR_RANGE);
      if (compact) *reinterpret_cast<uint32_t*>(reinterpret_cast<uint2*>(slots) + slot[u]) = LABEL_BIT32 | static_cast<uint32_t>(label);
      else slots[slot[u]].val = LABEL_BIT | static_cast<unsigned long long>(label);
      ++label;
    }
  }
}

// lookup: label of each id, -1 when absent
template <typename IdT>
__global__ void __launch_bounds__(RL_BLOCK)
relabel_lookup_kernel(const __grid_constant__ dgs_segments in, const int64_t n,
                      const Slot* __restrict__ slots, const uint64_t mask, const bool compact,
                      IdT* __restrict__ out) {
  pdl_enter();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * RL_BLOCK + threadIdx.x;
  if (i >= n) return;
  out[i] = static_cast<IdT>(probe_label(slots, mask, static_cast<long long>(seg_load<IdT>(in, i)), compact));
}

// lookup of the sequence with device-side counts, when it does not ride on another launch
template <typename IdT>
__global__ void __launch_bounds__(RL_BLOCK) relabel_lookup_pair_kernel(const LookupJob job) {
  pdl_enter();
  run_lookup_cta<IdT>(job, blockIdx.x);
}

inline int64_t seg_total(const dgs_segments& s) {
  int64_t t = 0;
  for (int i = 0; i < s.count; ++i) t += s.len[i];
  return t;
}

int check_segments(const dgs_segments* s, const char* who) {
  DGS_REQUIRE(s != nullptr && s->count >= 0 && s->count <= DGS_MAX_SEGMENTS, DGS_ERR_INVALID,
              "%s: bad segment list", who);
  for (int i = 0; i < s->count; ++i)
    DGS_REQUIRE(s->len[i] >= 0 && (s->len[i] == 0 || s->ptr[i] != nullptr), DGS_ERR_INVALID,
                "%s: segment %d is null", who, i);
  return DGS_OK;
}

__global__ void zero_word_kernel(int64_t* w) { *w = 0; }

// insert -> count -> number over a cleared table; n_bound sizes the grids
template <typename IdT, typename Keys>
int run_unique(const Keys& keys, Count n_keys, const TableSize& size, const TableView& t, void* unique_out,
               int64_t unique_capacity, int64_t* n_unique, const SizesReport& report, int32_t* status,
               cudaStream_t s) {
  const unsigned per_key_grid = static_cast<unsigned>((n_keys.bound + RL_BLOCK - 1) / RL_BLOCK);
  DGS_CUDA_TRY(launch_chained(SITE_INSERT, relabel_insert_kernel<IdT, Keys>, per_key_grid, RL_BLOCK, s, keys, size, t.slots,
                              t.slot_of, status));
  DGS_CUDA_TRY(launch_chained(SITE_COUNT, relabel_count_kernel, static_cast<unsigned>(t.ntiles), RL_BLOCK, s, n_keys, t.slots,
                              size.compact, t.slot_of, t.tile_off, t.ticket, t.total, n_unique, report));
  DGS_CUDA_TRY(launch_chained(SITE_NUMBER, relabel_number_kernel<IdT, Keys>, static_cast<unsigned>(t.ntiles), RL_BLOCK, s, keys,
                              t.slots, size.compact, t.slot_of, t.tile_off, static_cast<IdT*>(unique_out), unique_capacity,
                              status));
  return DGS_OK;
}

}  // namespace

int64_t* unique_total(void* table, int64_t key_bound) { return table_view(table, key_bound).total; }
unsigned int* unique_ticket(void* table, int64_t key_bound) { return table_view(table, key_bound).ticket; }

ClearJob make_clear_job(void* table, int64_t key_bound, const TableSize& size) {
  const TableView t = table_view(table, key_bound);
  return ClearJob{t.slots, size, static_cast<unsigned>((t.cap + CLEAR_SLOTS_PER_CTA - 1) / CLEAR_SLOTS_PER_CTA)};
}

LookupJob make_lookup_job(const void* table, int64_t key_bound, const TableSize& size, const void* a, const void* b,
                          Count n, void* out_a, void* out_b) {
  const TableView t = table_view(const_cast<void*>(table), key_bound);
  return LookupJob{a, b, out_a, out_b, n, t.slots, size, static_cast<unsigned>((n.bound + RL_BLOCK - 1) / RL_BLOCK)};
}

int launch_clear(const ClearJob& job, cudaStream_t s) {
  if (job.ctas == 0) return DGS_OK;
  DGS_CUDA_TRY(launch_chained(SITE_CLEAR, relabel_clear_kernel, job.ctas, RL_BLOCK, s, job));
  return DGS_OK;
}

int launch_unique_pair(bool ids64, const void* a, Count na, const void* b, Count nb, int64_t key_bound,
                       const TableSize& size, void* table, void* unique_out, int64_t unique_capacity,
                       int64_t* n_unique_out, const SizesReport& report, int32_t* status, cudaStream_t s) {
  DGS_REQUIRE(key_bound > 0 && key_bound < (1ll << 30) && na.bound + nb.bound <= key_bound, DGS_ERR_UNSUPPORTED,
              "relabel: %lld keys", (long long)key_bound);
  DGS_REQUIRE(na.dev != nullptr && nb.dev != nullptr && na.dev2 == nullptr && nb.dev2 == nullptr, DGS_ERR_INVALID,
              "relabel: the pair form takes one device word per length");
  const TableView t = table_view(table, key_bound);
  const Count n_keys{key_bound, na.dev, nb.dev};
  const PairKeys keys{a, b, na, nb};
  return ids64 ? run_unique<int64_t, PairKeys>(keys, n_keys, size, t, unique_out, unique_capacity, n_unique_out,
                                               report, status, s)
               : run_unique<int32_t, PairKeys>(keys, n_keys, size, t, unique_out, unique_capacity, n_unique_out,
                                               report, status, s);
}

int launch_lookup(const LookupJob& job, bool ids64, cudaStream_t s) {
  if (job.ctas == 0) return DGS_OK;
  if (ids64) DGS_CUDA_TRY(launch_chained(SITE_LOOKUP, relabel_lookup_pair_kernel<int64_t>, job.ctas, RL_BLOCK, s, job));
  else DGS_CUDA_TRY(launch_chained(SITE_LOOKUP, relabel_lookup_pair_kernel<int32_t>, job.ctas, RL_BLOCK, s, job));
  return DGS_OK;
}

}  // namespace dgs

extern "C" size_t dgs_relabel_table_bytes(int64_t n) {
  using namespace dgs;
  if (n < 0) n = 0;
  const int64_t ntiles = (n + RL_TILE - 1) / RL_TILE;
  return slots_for(n) * sizeof(Slot) + align_up(static_cast<size_t>(n) * sizeof(uint32_t), 16) +
         static_cast<size_t>(ntiles + 2) * sizeof(int64_t);
}

extern "C" int dgs_unique_first_occurrence(const dgs_segments* keys, int32_t ids64, void* table,
                                           size_t table_bytes, void* unique_out, int64_t* n_unique,
                                           int32_t* status, dgs_stream_t stream) {
  using namespace dgs;
  int rc = check_segments(keys, "dgs_unique_first_occurrence");
  if (rc != DGS_OK) return rc;
  const int64_t n = seg_total(*keys);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DGS_REQUIRE(table != nullptr && table_bytes >= dgs_relabel_table_bytes(n), DGS_ERR_INVALID,
              "dgs_unique_first_occurrence: table scratch too small (%zu < %zu)", table_bytes,
              dgs_relabel_table_bytes(n));
  DGS_REQUIRE((reinterpret_cast<uintptr_t>(table) & 15) == 0, DGS_ERR_INVALID,
              "dgs_unique_first_occurrence: table must be 16-byte aligned");
  DGS_REQUIRE(n < (1ll << 30), DGS_ERR_UNSUPPORTED, "dgs_unique_first_occurrence: %lld keys", (long long)n);
  const TableView t = table_view(table, n);
  if (n == 0) {
    DGS_CUDA_TRY(cudaMemsetAsync(t.slots, 0xFF, t.cap * sizeof(Slot), s));
    if (n_unique != nullptr) {
      zero_word_kernel<<<1, 1, 0, s>>>(n_unique);
      DGS_LAUNCH_CHECK();
    }
    return DGS_OK;
  }
  DGS_REQUIRE(unique_out != nullptr, DGS_ERR_INVALID, "dgs_unique_first_occurrence: null output");
  DGS_CUDA_TRY(cudaMemsetAsync(t.slots, 0xFF, t.cap * sizeof(Slot), s));
  DGS_CUDA_TRY(cudaMemsetAsync(t.ticket, 0, sizeof(unsigned int), s));
  const SegKeys sk{*keys, n};
  // 32-bit ids always fit the one-word slots; for 64-bit ids this entry point knows nothing about the id space
  const TableSize size{exact_count(n), 1, ids64 == 0};
  return ids64 ? run_unique<int64_t, SegKeys>(sk, exact_count(n), size, t, unique_out, n, n_unique, SizesReport{},
                                              status, s)
               : run_unique<int32_t, SegKeys>(sk, exact_count(n), size, t, unique_out, n, n_unique, SizesReport{},
                                              status, s);
}

extern "C" int dgs_relabel_lookup(const void* table, size_t table_bytes, int64_t n_keys_built,
                                  const dgs_segments* in, int32_t ids64, void* out,
                                  dgs_stream_t stream) {
  using namespace dgs;
  int rc = check_segments(in, "dgs_relabel_lookup");
  if (rc != DGS_OK) return rc;
  const int64_t n = seg_total(*in);
  if (n == 0) return DGS_OK;
  DGS_REQUIRE(table != nullptr && n_keys_built >= 0 && table_bytes >= dgs_relabel_table_bytes(n_keys_built),
              DGS_ERR_INVALID, "dgs_relabel_lookup: bad table");
  DGS_REQUIRE(out != nullptr, DGS_ERR_INVALID, "dgs_relabel_lookup: null output");
  DGS_REQUIRE((n + RL_BLOCK - 1) / RL_BLOCK <= 0x7fffffffLL, DGS_ERR_UNSUPPORTED, "dgs_relabel_lookup: too many ids");
  const TableView t = table_view(const_cast<void*>(table), n_keys_built);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((n + RL_BLOCK - 1) / RL_BLOCK);
  if (ids64)
    DGS_CUDA_TRY(launch_chained(SITE_LOOKUP, relabel_lookup_kernel<int64_t>, grid, RL_BLOCK, s, *in, n, t.slots, t.cap - 1,
                                false, static_cast<int64_t*>(out)));
  else  // the table of dgs_unique_first_occurrence for 32-bit ids has one-word slots
    DGS_CUDA_TRY(launch_chained(SITE_LOOKUP, relabel_lookup_kernel<int32_t>, grid, RL_BLOCK, s, *in, n, t.slots, t.cap - 1,
                                true, static_cast<int32_t*>(out)));
  return DGS_OK;
}
