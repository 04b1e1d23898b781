// Device-side pieces of the relabel table that more than one translation unit
// needs: the slot layout, the hash, and the two jobs (clearing a table, looking
// labels up) that the multi-hop sequence runs as extra CTAs of another kernel's
// launch instead of as launches of their own.
#pragma once
#include "common.cuh"

namespace dgs {

constexpr int RL_BLOCK = 256;
constexpr unsigned long long LABEL_BIT = 0x8000000000000000ull;
constexpr long long EMPTY_KEY = -1;  // cleared slot: key = -1, value = 2^64-1
constexpr uint32_t NO_SLOT = 0xFFFFFFFFu;
constexpr int CLEAR_SLOTS_PER_CTA = RL_BLOCK * 4;

struct __align__(16) Slot {
  long long key;
  unsigned long long val;
};

// Compact tables: when every key is below 2^32 - 1 (32-bit ids, or 64-bit ids of a graph with fewer nodes
// than that) a slot is ONE 64-bit word, key in the high half and the minimum input index (later the label)
// in the low half.  Claiming a slot and setting its first index is then a single compare-and-swap, a
// repeated key costs one load and at most one atomicMin, and every later pass reads 8 bytes per key instead
// of 16; the table (and the clearing of it) is half the size.  Input indices and labels stay below 2^30
// (the key count is limited to that), so bit 31 of the low half marks a label.  The same memory holds
// either form: a table laid out for `cap` 16-byte slots uses its first half as `cap` compact slots.
constexpr unsigned long long EMPTY_COMPACT = ~0ull;
constexpr uint32_t LABEL_BIT32 = 0x80000000u;
constexpr long long COMPACT_KEY_LIMIT = 0xFFFFFFFFll;  // keys must be below this

// slots in use for a table built for n keys: the power of two >= max(2n, 64)
__host__ __device__ __forceinline__ uint64_t slots_for(int64_t n) {
  uint64_t want = 2 * static_cast<uint64_t>(n);
  if (want < 64) want = 64;
#ifdef __CUDA_ARCH__
  return 1ull << (64 - __clzll(static_cast<long long>(want - 1)));
#else
  uint64_t cap = 64;
  while (cap < want) cap <<= 1;
  return cap;
#endif
}

// How many keys a table is dimensioned for: count_of(n) * mult.  The per-operator
// path knows its key count (mult = 1).  The multi-hop sequence dimensions a hop's
// table before that hop's neighbours are drawn, for seeds * (1 + fanout) keys.
struct TableSize {
  Count n;
  int64_t mult;
  bool compact;  // one-word slots (see above)
};

// Sizes that only the host needs (how much of each output is valid): device words copied to a
// host-visible array by the kernel that computes the last of them, so that a sequence of kernels
// pays for one write over the host link instead of one per size.
struct SizesReport {
  int64_t* dst;  // [n], pinned
  int n;         // 0: nothing to report
  const int64_t* src[2 * DGS_MAX_HOPS];
};

#ifdef __CUDACC__

__device__ __forceinline__ uint64_t table_slots(const TableSize& t) { return slots_for(count_of(t.n) * t.mult); }

__device__ __forceinline__ uint64_t hash_key(long long key) {
  uint64_t z = static_cast<uint64_t>(key);
  z = (z ^ (z >> 33)) * 0xFF51AFD7ED558CCDull;
  z = (z ^ (z >> 33)) * 0xC4CEB9FE1A85EC53ull;
  return z ^ (z >> 33);
}

// 32-bit finaliser for the one-word tables (their keys fit 32 bits and their slot counts stay below 2^31):
// a third of the instructions of the 64-bit mix, and these kernels are short of issue slots, not of bandwidth
__device__ __forceinline__ uint32_t hash_key32(uint32_t k) {
  k ^= k >> 16;
  k *= 0x85EBCA6Bu;
  k ^= k >> 13;
  k *= 0xC2B2AE35u;
  return k ^ (k >> 16);
}

__device__ __forceinline__ long long probe_label(const Slot* __restrict__ slots, uint64_t mask, long long key,
                                                 bool compact) {
  if (key < 0) return -1;
  if (compact) {
    if (key >= COMPACT_KEY_LIMIT) return -1;
    const unsigned long long* __restrict__ words = reinterpret_cast<const unsigned long long*>(slots);
    const uint32_t mask32 = static_cast<uint32_t>(mask), key32 = static_cast<uint32_t>(key);
    uint32_t h = hash_key32(key32) & mask32;
    for (uint32_t probes = 0; probes <= mask32; ++probes) {
      const uint2 w = reinterpret_cast<const uint2*>(words)[h];  // one 8-byte load: x = index / label, y = key
      if (w.y == key32) return static_cast<long long>(w.x & ~LABEL_BIT32);
      if ((w.x & w.y) == 0xFFFFFFFFu) break;                     // empty slot
      h = (h + 1) & mask32;
    }
    return -1;
  }
  uint64_t h = hash_key(key) & mask;
  for (uint64_t probes = 0; probes <= mask; ++probes) {
    const Slot s = slots[h];  // one 16-byte load
    if (s.key == key) return static_cast<long long>(s.val & ~LABEL_BIT);
    if (s.key == EMPTY_KEY) break;
    h = (h + 1) & mask;
  }
  return -1;
}

// ---- jobs that can ride on another kernel's launch -----------------------------
// Clear the slots a table will use.  Runs before anything touches the table.
struct ClearJob {
  Slot* slots;
  TableSize size;
  unsigned ctas;  // CLEAR_SLOTS_PER_CTA slots each; 0: no job
};
__device__ __forceinline__ void run_clear_cta(const ClearJob& j, unsigned cta) {
  // in 16-byte units: compact slots are half as wide
  const uint64_t cap = j.size.compact ? table_slots(j.size) / 2 : table_slots(j.size);
  const uint64_t i = static_cast<uint64_t>(cta) * CLEAR_SLOTS_PER_CTA + threadIdx.x;
  const ulonglong2 empty = make_ulonglong2(~0ull, ~0ull);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const uint64_t at = i + static_cast<uint64_t>(u) * RL_BLOCK;
    if (at < cap) *reinterpret_cast<ulonglong2*>(&j.slots[at]) = empty;
  }
}

// Relabel a finished hop's COO: out_a[i] = label(a[i]) (skipped when a is null),
// out_b[i] = label(b[i]), i < n; in place is fine.  Needs that hop's numbering.
struct LookupJob {
  const void* a;
  const void* b;
  void* out_a;
  void* out_b;
  Count n;
  const Slot* slots;
  TableSize size;
  unsigned ctas;  // RL_BLOCK ids each; 0: no job
};
template <typename IdT>
__device__ __forceinline__ void run_lookup_cta(const LookupJob& j, unsigned cta) {
  const int64_t i = static_cast<int64_t>(cta) * RL_BLOCK + threadIdx.x;
  // the ids are read while the live count and the table size are still on their way (room for n.bound ids)
  const bool in_bound = i < j.n.bound;
  const long long ka = (in_bound && j.a != nullptr) ? static_cast<long long>(static_cast<const IdT*>(j.a)[i]) : -1;
  const long long kb = in_bound ? static_cast<long long>(static_cast<const IdT*>(j.b)[i]) : -1;
  if (i >= count_of(j.n)) return;
  const uint64_t mask = table_slots(j.size) - 1;
  if (j.a != nullptr) static_cast<IdT*>(j.out_a)[i] = static_cast<IdT>(probe_label(j.slots, mask, ka, j.size.compact));
  static_cast<IdT*>(j.out_b)[i] = static_cast<IdT>(probe_label(j.slots, mask, kb, j.size.compact));
}

#endif  // __CUDACC__
}  // namespace dgs
