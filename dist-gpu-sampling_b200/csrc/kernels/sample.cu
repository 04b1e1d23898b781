// Row-wise neighbour sampling on a CSC graph whose indptr / indices / weights
// live in ChunkTensors (or plain device tensors: num_parts == 1).
//
// Replaces, for both the plain-tensor and the ChunkTensor operators:
//   _GetSubIndptr + cub scan + blocking nnz read-back
//       (reference src/cuda/rowwise_sampling.cu:13-40,147),
//   _CSRRowWiseSampleUniformKernel / ...ReplaceKernel
//       (src/cuda/rowwise_sampling.cu:42-136,
//        src/cuda/rowwise_sampling_with_chunk_tensor.cu:15-111),
//   _CSRRowWiseSampleKernel / ...ReplaceKernel (weighted)
//       (src/cuda/rowwise_sampling_probs.cu:54-216) and the faiss-derived
//       WarpSelect it uses (src/cuda/warpselect/*.cuh).
//
// What is kept (the contract): per-seed counts min(deg,k) / (deg?k:0); COO
// grouped by seed position; rows with deg <= k copied whole in CSC order;
// uniform k-subsets / A-Res weighted subsets / proportional draws otherwise.
//
// What is different (the design):
//   * the reference spends one 128-thread block and one curand_init per seed
//     and draws O(deg) random numbers per row (Algorithm R).  Here a seed gets
//     a sub-warp group of G = 4..32 lanes (G >= k), the row is never scanned:
//     k candidate positions are drawn at once with counter-based Philox and
//     duplicates are re-drawn until the k positions are distinct
//     (__match_any_sync across the warp).  Equal treatment of positions makes
//     every k-subset equally likely.  When k > deg/2 the deg-k positions to
//     LEAVE OUT are drawn instead, so a draw collides with probability < 1/2.
//   * bounded integers use Lemire's multiply-shift with rejection instead of
//     `rand % n`.
//   * weighted sampling without replacement keeps the top-k keys in a sorted
//     per-warp register list (lane i = i-th largest) with ballot-gated
//     insertion; keys are compared in the log domain, log(u)/w, which orders
//     exactly like u^(1/w) but does not underflow for small weights.  Rows
//     are read in 512-edge windows (16 loads in flight per lane) and rows longer
//     than 4096 edges are shared by the eight warps of the CTA and merged.
//   * weighted sampling with replacement builds no cumulative array in global
//     memory: the row is streamed twice through a warp scan and each draw is
//     resolved by a ballot in the 32-edge window it falls into.
//   * counts, offsets and the total come from ONE plan kernel: every CTA scans
//     its 256 seeds and the CTA that finishes last (an atomic ticket, nobody
//     waits) scans the per-tile sums; the total goes to a caller-supplied
//     (pinned) word, so the host learns the output size while the sampling
//     kernel is still running.
//   * the sampling kernels give every seed its own group / warp and never loop
//     over seeds, so even a 1 024-seed hop fills the machine with independent
//     short chains instead of a few long ones.
#include "common.cuh"
#include "launchers.h"
#include "philox.cuh"
#include "tile_scan.cuh"

namespace dgs {
namespace {

constexpr int SAMPLE_TILE = 256;   // seeds per CTA
constexpr int SAMPLE_BLOCK = 256;  // threads per CTA

constexpr uint32_t TAG_UNIFORM = 0x554E4931u;
constexpr uint32_t TAG_REPLACE = 0x5245504Cu;
constexpr uint32_t TAG_FLOYD = 0x464C4F59u;
constexpr uint32_t TAG_ARES = 0x41524553u;
constexpr uint32_t TAG_WREPL = 0x57524550u;

struct PlanView {
  int64_t* row_begin;  // [n]
  int64_t* deg;        // [n]
  int64_t* local_off;  // [n]       exclusive prefix of the counts inside the seed's 256-tile
  int64_t* tile_off;   // [ntiles]  per-tile sums, scanned in place by the last CTA
  int64_t* total;      // [1]
  unsigned int* ticket;  // [1]     CTAs that have published their tile sum
  int64_t ntiles;
};

inline PlanView plan_view(void* plan, int64_t n) {
  PlanView v;
  v.ntiles = (n + SAMPLE_TILE - 1) / SAMPLE_TILE;
  v.row_begin = static_cast<int64_t*>(plan);
  v.deg = v.row_begin + n;
  v.local_off = v.deg + n;
  v.tile_off = v.local_off + n;
  v.total = v.tile_off + v.ntiles;
  v.ticket = reinterpret_cast<unsigned int*>(v.total + 1);
  return v;
}

__device__ __forceinline__ int64_t pick_count(int64_t deg, int64_t k, bool replace) {
  return replace ? (deg > 0 ? k : 0) : (deg < k ? deg : k);
}

// ---------------------------------------------------------------------------
// plan: row range per seed + per-tile output counts
// ---------------------------------------------------------------------------
template <typename IdT>
__global__ void __launch_bounds__(SAMPLE_BLOCK)
sample_plan_kernel(const __grid_constant__ dgs_chunk_desc indptr, const IdT* __restrict__ seeds,
                   const Count nc, const int64_t k, const bool replace,
                   int64_t* __restrict__ row_begin, int64_t* __restrict__ deg_out,
                   int64_t* __restrict__ local_off, int64_t* tile_sums, int64_t* total_out,
                   unsigned int* ticket, int64_t* nnz_out, const unsigned int plan_tiles,
                   const ClearJob clear, const LookupJob lookup, int32_t* __restrict__ status) {
  __shared__ int64_t smem[SAMPLE_BLOCK / 32 + 1];
  constexpr int sh = sizeof(IdT) == 8 ? 3 : 2;
  pdl_enter();
  if (blockIdx.x >= plan_tiles) {  // CTAs beyond the plan's tiles carry the independent jobs
    const unsigned int extra = blockIdx.x - plan_tiles;
    if (extra < clear.ctas) run_clear_cta(clear, extra);
    else run_lookup_cta<IdT>(lookup, extra - clear.ctas);
    return;
  }
  const int64_t i = static_cast<int64_t>(blockIdx.x) * SAMPLE_TILE + threadIdx.x;
  // the seed is read before the live count arrives (the list has room for nc.bound entries), so that
  // the two round trips overlap; an entry past the count is never used
  const IdT seed_raw = i < nc.bound ? seeds[i] : IdT(0);
  const int64_t n = count_of(nc);
  const int64_t s = static_cast<int64_t>(seed_raw);
  const bool good = i < n && s >= 0 && s + 1 < indptr.total;
  if (i < n && !good) raise_status(status, DGS_ERR_RANGE);
  // indptr[s] and indptr[s + 1] are fetched by TWO NEIGHBOURING LANES in one load instruction, half a warp's
  // seeds at a time: the two addresses (almost always) lie in the same 128-byte line, so the pair costs one
  // memory request instead of the two that two loads of one thread cost.  Inside one GPU that is noise; when
  // the row of indptr lives on a peer, requests are what the link can deliver only so many of per second.
  const int lane = threadIdx.x & 31;
  int64_t pair[2] = {0, 0};  // this lane's (row begin, row end) after the two half-warp passes
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int owner = half * 16 + (lane >> 1);  // the lane whose seed this lane fetches an element for
    const int64_t so = __shfl_sync(FULL_MASK, s, owner);
    const bool ok = __shfl_sync(FULL_MASK, good ? 1 : 0, owner) != 0;
    const int64_t v = ok ? static_cast<int64_t>(load_at<IdT>(indptr, sh, so + (lane & 1))) : 0;
    const int64_t lo = __shfl_sync(FULL_MASK, v, 2 * (lane & 15));
    const int64_t hi = __shfl_sync(FULL_MASK, v, 2 * (lane & 15) + 1);
    if ((lane >> 4) == half) {
      pair[0] = lo;
      pair[1] = hi;
    }
  }
  int64_t cnt = 0;
  if (i < n) {
    int64_t rb = 0, deg = 0;
    if (good) {
      rb = pair[0];
      deg = pair[1] - rb;
      if (deg < 0 || rb < 0) {
        raise_status(status, DGS_ERR_RANGE);
        deg = 0;
        rb = 0;
      }
    }
    row_begin[i] = rb;
    deg_out[i] = deg;
    cnt = pick_count(deg, k, replace);
  }
  int64_t total;
  const int64_t ex = block_exclusive_scan<int64_t, SAMPLE_BLOCK>(cnt, smem, &total);
  if (i < n) local_off[i] = ex;

  // publish the tile sum; the CTA that draws the last ticket scans all of them
  publish_and_scan_tiles<SAMPLE_BLOCK>(total, tile_sums, ticket, total_out, nnz_out, smem, plan_tiles);
}

// ---------------------------------------------------------------------------
// shared pieces of the sampling kernels
// ---------------------------------------------------------------------------
template <typename IdT>
struct Emit {
  const dgs_chunk_desc& indices;
  IdT* coo_row;
  IdT* coo_col;
  int64_t* picked_pos;
  int64_t out_capacity;
  int32_t* status;

  // t-th output of a seed whose outputs start at o; `pos` = position in its row
  __device__ __forceinline__ void operator()(int64_t o, int64_t t, int64_t seed, int64_t rb,
                                             int64_t pos) const {
    constexpr int sh = sizeof(IdT) == 8 ? 3 : 2;
    const int64_t at = o + t;
    if (at >= out_capacity) {
      raise_status(status, DGS_ERR_RANGE);
      return;
    }
    const int64_t e = rb + pos;
    IdT c = static_cast<IdT>(-1);
    if (e >= 0 && e < indices.total) c = load_at<IdT>(indices, sh, e);
    else raise_status(status, DGS_ERR_RANGE);
    coo_row[at] = static_cast<IdT>(seed);
    coo_col[at] = c;
    if (picked_pos != nullptr) picked_pos[at] = pos;
  }
};

// What a group / warp needs to know about its seed.
struct SeedPlan {
  int64_t rb, deg, o;
};
__device__ __forceinline__ SeedPlan seed_plan(const int64_t* __restrict__ plan_rb,
                                              const int64_t* __restrict__ plan_deg,
                                              const int64_t* __restrict__ local_off,
                                              const int64_t* __restrict__ tile_off, int64_t i, bool valid) {
  SeedPlan p{0, 0, 0};
  if (valid) {
    p.rb = plan_rb[i];
    p.deg = plan_deg[i];
    p.o = tile_off[i / SAMPLE_TILE] + local_off[i];
  }
  return p;
}

// ---------------------------------------------------------------------------
// uniform sampling: G lanes per seed
// ---------------------------------------------------------------------------
template <typename IdT, int G>
__global__ void __launch_bounds__(SAMPLE_BLOCK, 6)
sample_uniform_kernel(const __grid_constant__ dgs_chunk_desc indices, const IdT* __restrict__ seeds,
                      const Count nc, const int64_t k, const bool replace,
                      const int64_t* __restrict__ plan_rb, const int64_t* __restrict__ plan_deg,
                      const int64_t* __restrict__ local_off, const int64_t* __restrict__ tile_off,
                      const RngKey rng, IdT* coo_row, IdT* coo_col,
                      const int64_t out_capacity, int64_t* __restrict__ picked_pos,
                      const bool row_is_position, int32_t* __restrict__ status) {
  const Emit<IdT> emit{indices, coo_row, coo_col, picked_pos, out_capacity, status};
  pdl_enter();
  const uint64_t key = key_of(rng);
  constexpr int GROUPS = SAMPLE_BLOCK / G;  // seeds per CTA
  constexpr int TAKEN_WORDS = 4096;         // 16 KB of position bitmaps per CTA, split between its groups
  __shared__ uint32_t s_taken[TAKEN_WORDS];
  const int lane = threadIdx.x & 31;
  const int l = threadIdx.x % G;        // lane inside the group
  const int group = threadIdx.x / G;    // group inside the CTA
  const int gw = lane / G;              // group inside the warp
  const unsigned gmask = (G == 32) ? FULL_MASK : (((1u << G) - 1u) << (gw * G));
  const bool fast = !replace && k <= G;  // uniform over the grid

  {  // one seed per group; all 32 lanes of a warp walk through the same code
    const int64_t slot = static_cast<int64_t>(blockIdx.x) * GROUPS + group;
    // everything that only needs the slot is read before the live count arrives (all arrays have room for
    // nc.bound entries); what belongs to a slot past the count is dropped below
    const bool in_bound = slot < nc.bound;
    const int64_t i = slot;  // the seed this group serves
    const SeedPlan sp = seed_plan(plan_rb, plan_deg, local_off, tile_off, i, in_bound);
    const int64_t seed_raw = !in_bound ? 0 : (row_is_position ? i : static_cast<int64_t>(seeds[i]));
    const bool valid = slot < count_of(nc);
    const int64_t deg = valid ? sp.deg : 0, rb = valid ? sp.rb : 0, o = valid ? sp.o : 0;
    const int64_t seed = valid ? seed_raw : 0;
    const uint32_t i_lo = static_cast<uint32_t>(i), i_hi = static_cast<uint32_t>(static_cast<uint64_t>(i) >> 32);

    if (replace) {
      if (valid && deg > 0)
        for (int64_t t = l; t < k; t += G) {
          const Philox4 r = philox4x32_10(key, i_lo, i_hi, static_cast<uint32_t>(t), TAG_REPLACE);
          emit(o, t, seed, rb, static_cast<int64_t>(bounded(r, static_cast<uint64_t>(deg))));
        }
      return;
    }

    if (fast) {
      // -- distinct positions by parallel rejection (all 32 lanes take part) --
      // Every lane of a group draws a position and marks it in the group's bitmap
      // in shared memory; a lane that finds its bit already set draws again.  Only
      // equality of positions matters, so every k-subset is equally likely.
      constexpr int WORDS = TAKEN_WORDS / GROUPS;         // bitmap words per group
      constexpr int64_t MAP_DEG = static_cast<int64_t>(WORDS) * 32;
      uint32_t* taken = s_taken + group * WORDS;
      const bool sampled = valid && deg > k;
      const bool complement = sampled && 2 * k > deg;  // draw the deg-k positions to leave out
      const int64_t m = sampled ? (complement ? deg - k : k) : 0;
      const bool active = l < m;
      const bool in_map = deg <= MAP_DEG;              // longer rows compare candidates across the warp
      if (sampled && in_map)
        for (int wd = l; wd < static_cast<int>((deg + 31) >> 5); wd += G) taken[wd] = 0u;
      __syncwarp();
      bool need = active;
      int64_t c = 0;
      const bool small_row = deg <= 0xFFFFFFFFll;  // every real graph; longer rows take the general path
      const uint32_t deg32 = static_cast<uint32_t>(deg);
      Philox4 rnd{0u, 0u, 0u, 0u};
      for (uint32_t round = 0; __any_sync(FULL_MASK, need); ++round) {
        // one Philox block per lane feeds four rounds of (re)draws
        if ((round & 3u) == 0u && active && round < 64)
          rnd = philox4x32_10(key, i_lo, i_hi, ((round >> 2) << 8) | static_cast<uint32_t>(l), TAG_UNIFORM);
        bool usable = true;  // false: this attempt hit Lemire's rejection zone, draw again next round
        if (need) {
          if (round >= 64) {  // never reached in practice: step to a neighbour, keeps the loop bounded
            c = (c + 1 == deg) ? 0 : c + 1;
          } else if (small_row) {
            const uint32_t word = (round & 2u) ? ((round & 1u) ? rnd.w : rnd.z) : ((round & 1u) ? rnd.y : rnd.x);
            uint32_t pick;
            usable = bounded_try(word, deg32, &pick);
            c = pick;
          } else {
            const Philox4 r = philox4x32_10(key, i_lo, i_hi, (round << 8) | static_cast<uint32_t>(l), TAG_UNIFORM ^ 1u);
            c = static_cast<int64_t>(bounded(r, static_cast<uint64_t>(deg)));
          }
          if (in_map && usable) {
            const uint32_t bit = 1u << (static_cast<uint32_t>(c) & 31u);
            need = (atomicOr(&taken[c >> 5], bit) & bit) != 0u;
          }
        }
        if (__any_sync(FULL_MASK, active && !in_map)) {
          // lanes holding the same position inside one group see each other; the lowest keeps it
          const bool mine = active && !in_map;
          const unsigned long long tag =
              (mine && usable) ? (static_cast<unsigned long long>(c) | (static_cast<unsigned long long>(gw) << 58))
                               : (0x8000000000000000ull | static_cast<unsigned long long>(lane));
          const unsigned same = __match_any_sync(FULL_MASK, tag);
          if (mine) need = !usable || (__ffs(same) - 1 != lane);
        }
        if (round >= 64 + 1024) {
          if (need) raise_status(status, DGS_ERR_TABLE_FULL);
          break;
        }
      }
      __syncwarp();
      if (complement) {
        // the row has at most 2k-1 <= 63 positions, so its bitmap is one or two words:
        // every lane ranks its own two positions (a = l and b = l + G cover the row)
        // among the kept ones
        const unsigned long long out_mask =
            static_cast<unsigned long long>(taken[0]) |
            (deg > 32 ? static_cast<unsigned long long>(taken[1]) << 32 : 0ull);
        const unsigned long long row_mask = (1ull << deg) - 1ull;  // deg <= 63
        const unsigned long long kept = ~out_mask & row_mask;
        const int a = l, b = l + G;
        if ((kept >> a) & 1ull) emit(o, __popcll(kept & ((1ull << a) - 1ull)), seed, rb, a);
        if (b < 64 && ((kept >> b) & 1ull)) emit(o, __popcll(kept & ((1ull << b) - 1ull)), seed, rb, b);
      }
      if (sampled && !complement) {
        if (active) emit(o, l, seed, rb, c);
      } else if (valid && !sampled) {
        if (l < deg) emit(o, l, seed, rb, l);  // whole row, CSC order (deg <= k <= G)
      }
      return;
    }

    // -- general k (> G is only possible with G == 32: the group is the warp) --
    if (!valid) return;
    if (deg <= k) {
      for (int64_t t = l; t < deg; t += G) emit(o, t, seed, rb, t);
    } else if (o + k > out_capacity) {
      if (l == 0) raise_status(status, DGS_ERR_RANGE);
    } else {
      // Floyd's subset algorithm; the chosen positions are parked in coo_col
      volatile IdT* slots = coo_col + o;
      int64_t have = 0;
      for (int64_t j = deg - k; j < deg; ++j, ++have) {
        const Philox4 r = philox4x32_10(key, i_lo, i_hi, static_cast<uint32_t>(have), TAG_FLOYD);
        const int64_t t = static_cast<int64_t>(bounded(r, static_cast<uint64_t>(j + 1)));
        bool found = false;
        for (int64_t q = l; q < have; q += G) found |= (static_cast<int64_t>(slots[q]) == t);
        found = __any_sync(gmask, found);
        if (l == 0) slots[have] = static_cast<IdT>(found ? j : t);
        __syncwarp(gmask);
      }
      for (int64_t q = l; q < k; q += G) emit(o, q, seed, rb, static_cast<int64_t>(slots[q]));
    }
  }
}

// ---------------------------------------------------------------------------
// weighted sampling: one warp per seed; rows longer than HUB_DEG edges are then
// taken on by all eight warps of the CTA together
// ---------------------------------------------------------------------------
struct RowWeights {
  const dgs_chunk_desc& probs;
  const float* direct;  // non-null when the whole row lies in one storage region
  int64_t rb;
  __device__ __forceinline__ float operator()(int64_t e) const {
    return direct != nullptr ? direct[e] : load_at<float>(probs, 2, rb + e);
  }
};

constexpr int64_t HUB_DEG = 4096;   // rows above this are scanned by the whole CTA
constexpr int ARES_QUADS = 4;       // Philox blocks per lane and 512-edge window

// The running top-k of one warp: lane j holds the j-th largest key and its
// position in the row; `thresh` is the key held by lane k-1 (the entry bar).
struct TopK {
  float key;
  int64_t pos;
  float thresh;
  __device__ __forceinline__ void insert(float nk, int64_t np, int l, int k) {
    // warp-uniform call with nk > thresh; the keys >= nk form a prefix of the lanes
    const int p = __popc(__ballot_sync(FULL_MASK, key >= nk));  // p <= k-1
    const float up_key = __shfl_up_sync(FULL_MASK, key, 1);
    const int64_t up_pos = __shfl_up_sync(FULL_MASK, pos, 1);
    if (l > p) {
      key = up_key;
      pos = up_pos;
    } else if (l == p) {
      key = nk;
      pos = np;
    }
    thresh = __shfl_sync(FULL_MASK, key, k - 1);
  }
};

// A-Res over one window of 512 edges starting at `base`: key = log(u)/w, which
// orders like u^(1/w).  The 16 weights a lane needs are loaded together (2 KB in
// flight per warp); the uniforms come from one Philox block per four edges,
// addressed by (seed position, edge index) so that the result does not depend on
// which warp scans the window.
__device__ __forceinline__ void ares_window(TopK& top, const RowWeights& W, int64_t base, int64_t deg,
                                            uint64_t key, uint32_t i_lo, uint32_t i_hi, int l, int k) {
  const float NEG_INF = __int_as_float(0xff800000);
  const float FLOOR_ZERO_W = -3.402823466e+38f;  // weight <= 0: behind every positive weight
  const float FLOOR_POS_W = -3.0e+38f;           // clamp for positive weights
  float wv[4 * ARES_QUADS];
#pragma unroll
  for (int j = 0; j < 4 * ARES_QUADS; ++j) {
    const int64_t e = base + j * 32 + l;
    wv[j] = (e < deg) ? W(e) : 0.f;
  }
#pragma unroll
  for (int q = 0; q < ARES_QUADS; ++q) {
    if (base + q * 128 >= deg) break;  // warp-uniform
    const uint64_t ctr = static_cast<uint64_t>((base >> 2) + q * 32) + static_cast<uint64_t>(l);
    const Philox4 r = philox4x32_10(key ^ (static_cast<uint64_t>(TAG_ARES) << 32), i_lo, i_hi,
                                    static_cast<uint32_t>(ctr), static_cast<uint32_t>(ctr >> 32));
    const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t e0 = base + (q * 4 + j) * 32;  // first edge of this group of 32
      const float w = wv[q * 4 + j];
      float ck = NEG_INF;
      if (e0 + l < deg)
        ck = (w > 0.f) ? fmaxf(__fdividef(__logf(unit_float(rw[j])), w), FLOOR_POS_W) : FLOOR_ZERO_W;
      unsigned cand = __ballot_sync(FULL_MASK, ck > top.thresh);
      while (cand) {
        const int src = __ffs(cand) - 1;
        cand &= cand - 1;
        const float nk = __shfl_sync(FULL_MASK, ck, src);
        if (nk > top.thresh) top.insert(nk, e0 + src, l, k);  // the bar may have risen since the ballot
      }
    }
  }
}

// One warp's share of a row: windows base0, base0 + stride, ...
// (The exponential-jump form of the sampler -- keys only for the edges that enter, a
// streamed prefix sum for the rest -- was built and measured here: with fan-outs of
// 10-32 and rows of 10^3-10^4 edges an entry costs ~250 instructions at a rate of k/n
// per edge, and the kernel ran 1.6-2.3x slower than with per-edge keys, so it is not used.)
__device__ __forceinline__ void ares_scan(TopK& top, const RowWeights& W, int64_t base0, int64_t stride,
                                          int64_t deg, uint64_t key, uint32_t i_lo, uint32_t i_hi, int l, int k) {
  for (int64_t base = base0; base < deg; base += stride) ares_window(top, W, base, deg, key, i_lo, i_hi, l, k);
}

template <typename IdT>
__global__ void __launch_bounds__(SAMPLE_BLOCK)
sample_weighted_kernel(const __grid_constant__ dgs_chunk_desc indices,
                       const __grid_constant__ dgs_chunk_desc probs, const IdT* __restrict__ seeds,
                       const Count nc, const int64_t k, const bool replace,
                       const int64_t* __restrict__ plan_rb, const int64_t* __restrict__ plan_deg,
                       const int64_t* __restrict__ local_off, const int64_t* __restrict__ tile_off,
                       const RngKey rng, IdT* coo_row, IdT* coo_col,
                       const int64_t out_capacity, int64_t* __restrict__ picked_pos,
                       const bool row_is_position, int32_t* __restrict__ status) {
  const Emit<IdT> emit{indices, coo_row, coo_col, picked_pos, out_capacity, status};
  pdl_enter();
  const uint64_t key = key_of(rng);
  const int64_t n = count_of(nc);
  const int l = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  constexpr int WARPS = SAMPLE_BLOCK / 32;
  const float NEG_INF = __int_as_float(0xff800000);
  __shared__ int s_hub[WARPS];  // warps whose seed is left to the whole CTA
  __shared__ int s_nhub;
  __shared__ float s_mkey[WARPS][32];
  __shared__ int64_t s_mpos[WARPS][32];
  if (threadIdx.x == 0) s_nhub = 0;
  __syncthreads();

  // ---- phase 1: one seed per warp ----
  do {
    const int64_t slot = static_cast<int64_t>(blockIdx.x) * WARPS + warp;
    if (slot >= n) break;  // warp-uniform
    const int64_t i = slot;
    const SeedPlan sp = seed_plan(plan_rb, plan_deg, local_off, tile_off, i, true);
    const int64_t deg = sp.deg, rb = sp.rb, o = sp.o;
    const int64_t seed = row_is_position ? i : static_cast<int64_t>(seeds[i]);
    const uint32_t i_lo = static_cast<uint32_t>(i), i_hi = static_cast<uint32_t>(static_cast<uint64_t>(i) >> 32);
    if (deg <= 0) break;

    if (!replace && deg <= k) {
      for (int64_t t = l; t < deg; t += 32) emit(o, t, seed, rb, t);
      break;
    }
    if (rb + deg > probs.total) {
      if (l == 0) raise_status(status, DGS_ERR_RANGE);
      break;
    }
    if (!replace && deg > HUB_DEG) {
      if (l == 0) s_hub[atomicAdd(&s_nhub, 1)] = warp;
      break;
    }
    int64_t run;
    const char* wp = resolve(probs, 2, rb, &run);
    const RowWeights W{probs, run >= deg ? reinterpret_cast<const float*>(wp) : nullptr, rb};

    if (!replace) {
      TopK top{NEG_INF, -1, NEG_INF};
      ares_scan(top, W, 0, 128 * ARES_QUADS, deg, key, i_lo, i_hi, l, static_cast<int>(k));
      if (l < k) emit(o, l, seed, rb, top.pos);
    } else {
      // ---- proportional draws: stream the row twice through a warp scan ----
      float total = 0.f;
      for (int64_t base = 0; base < deg; base += 32) {
        const int64_t e = base + l;
        float w = (e < deg) ? fmaxf(W(e), 0.f) : 0.f;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const float t = __shfl_up_sync(FULL_MASK, w, d);
          if (l >= d) w += t;
        }
        total = __shfl_sync(FULL_MASK, total + w, 31);
      }
      for (int64_t t0 = 0; t0 < k; t0 += 32) {
        const int64_t t = t0 + l;
        const bool mine = t < k;
        const Philox4 r = philox4x32_10(key, i_lo, i_hi, static_cast<uint32_t>(t), TAG_WREPL);
        const float draw = unit_float(r.x) * total;
        bool done = !mine;
        int64_t pos = deg - 1;  // a draw not below the final sum maps to the last edge
        float carry = 0.f;
        for (int64_t base = 0; base < deg; base += 32) {
          const int64_t e = base + l;
          float w = (e < deg) ? fmaxf(W(e), 0.f) : 0.f;
#pragma unroll
          for (int d = 1; d < 32; d <<= 1) {
            const float x = __shfl_up_sync(FULL_MASK, w, d);
            if (l >= d) w += x;
          }
          const float cdf = carry + w;  // inclusive prefix up to edge e
          const float window_end = __shfl_sync(FULL_MASK, cdf, 31);
          unsigned hit = __ballot_sync(FULL_MASK, !done && draw < window_end);
          while (hit) {
            const int src = __ffs(hit) - 1;
            hit &= hit - 1;
            const float d0 = __shfl_sync(FULL_MASK, draw, src);
            const unsigned above = __ballot_sync(FULL_MASK, cdf > d0);  // non-empty: lane 31 is above
            if (l == src) {
              int64_t q = base + (__ffs(above) - 1);
              pos = q < deg ? q : deg - 1;
              done = true;
            }
          }
          carry = window_end;
          if (__all_sync(FULL_MASK, done)) break;
        }
        if (mine) emit(o, t, seed, rb, pos);
      }
    }
  } while (false);

  // ---- phase 2: hub rows, all warps of the CTA on one row at a time ----
  __syncthreads();
  const int nhub = s_nhub;
  for (int h = 0; h < nhub; ++h) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * WARPS + s_hub[h];
    const SeedPlan sp = seed_plan(plan_rb, plan_deg, local_off, tile_off, i, true);
    const int64_t deg = sp.deg, rb = sp.rb, o = sp.o;
    const uint32_t i_lo = static_cast<uint32_t>(i), i_hi = static_cast<uint32_t>(static_cast<uint64_t>(i) >> 32);
    int64_t run;
    const char* wp = resolve(probs, 2, rb, &run);
    const RowWeights W{probs, run >= deg ? reinterpret_cast<const float*>(wp) : nullptr, rb};
    TopK top{NEG_INF, -1, NEG_INF};
    ares_scan(top, W, static_cast<int64_t>(warp) * 128 * ARES_QUADS, 128 * ARES_QUADS * WARPS, deg, key, i_lo,
              i_hi, l, static_cast<int>(k));
    s_mkey[warp][l] = top.key;
    s_mpos[warp][l] = top.pos;
    __syncthreads();
    if (warp == 0) {  // merge the other warps' lists into this one; every list is sorted, so stop at the bar
      for (int ww = 1; ww < WARPS; ++ww)
        for (int t = 0; t < k; ++t) {
          const float nk = s_mkey[ww][t];  // same address for all lanes: broadcast
          if (!(nk > top.thresh)) break;
          top.insert(nk, s_mpos[ww][t], l, static_cast<int>(k));
        }
      if (l < k) emit(o, l, row_is_position ? i : static_cast<int64_t>(seeds[i]), rb, top.pos);
    }
    __syncthreads();
  }
}

__global__ void copy_total_kernel(const int64_t* total, int64_t* nnz) { *nnz = *total; }
__global__ void zero_total_kernel(int64_t* nnz) { *nnz = 0; }

int check_sample_args(const char* who, const void* seeds, int64_t n, int64_t k, const void* plan) {
  DGS_REQUIRE(n >= 0 && k >= 0, DGS_ERR_INVALID, "%s: n=%lld k=%lld", who, (long long)n, (long long)k);
  DGS_REQUIRE(n == 0 || (seeds != nullptr && plan != nullptr), DGS_ERR_INVALID, "%s: null buffer", who);
  DGS_REQUIRE(n / (SAMPLE_BLOCK / 32) < 0x7fffffffLL, DGS_ERR_UNSUPPORTED, "%s: too many seeds", who);
  return DGS_OK;
}

template <typename IdT>
int plan_typed(const dgs_chunk_desc& indptr, const void* seeds, Count n, int64_t k, bool replace,
               const PlanView& pv, int64_t* nnz, const ClearJob& clear, const LookupJob& lookup, int32_t* status,
               cudaStream_t s) {
  const unsigned tiles = static_cast<unsigned>(pv.ntiles);
  DGS_CUDA_TRY(launch_chained(SITE_PLAN, sample_plan_kernel<IdT>, tiles + clear.ctas + lookup.ctas, SAMPLE_BLOCK, s, indptr,
                              static_cast<const IdT*>(seeds), n, k, replace, pv.row_begin, pv.deg, pv.local_off,
                              pv.tile_off, pv.total, pv.ticket, nnz, tiles, clear, lookup, status));
  return DGS_OK;
}

template <typename IdT>
int uniform_typed(const dgs_chunk_desc& indices, const void* seeds, Count n, int64_t k, bool replace,
                  const PlanView& pv, RngKey key, void* coo_row, void* coo_col,
                  int64_t cap, int64_t* pos, bool rowpos, int32_t* status, cudaStream_t s) {
#define DGS_LAUNCH_U(G)                                                                                      \
  DGS_CUDA_TRY(launch_chained(SITE_SAMPLE, sample_uniform_kernel<IdT, G>,                                                 \
                              static_cast<unsigned>((n.bound + SAMPLE_BLOCK / G - 1) / (SAMPLE_BLOCK / G)),  \
                              SAMPLE_BLOCK, s, indices, static_cast<const IdT*>(seeds), n, k, replace,       \
                              pv.row_begin, pv.deg, pv.local_off, pv.tile_off, key,                          \
                              static_cast<IdT*>(coo_row), static_cast<IdT*>(coo_col), cap, pos, rowpos, status))
  if (k <= 4) DGS_LAUNCH_U(4);
  else if (k <= 8) DGS_LAUNCH_U(8);
  else if (k <= 16) DGS_LAUNCH_U(16);
  else DGS_LAUNCH_U(32);
#undef DGS_LAUNCH_U
  return DGS_OK;
}

template <typename IdT>
int weighted_typed(const dgs_chunk_desc& indices, const dgs_chunk_desc& probs, const void* seeds, Count n,
                   int64_t k, bool replace, const PlanView& pv, RngKey key,
                   void* coo_row, void* coo_col, int64_t cap, int64_t* pos, bool rowpos, int32_t* status,
                   cudaStream_t s) {
  const unsigned grid = static_cast<unsigned>((n.bound + SAMPLE_BLOCK / 32 - 1) / (SAMPLE_BLOCK / 32));
  DGS_CUDA_TRY(launch_chained(SITE_SAMPLE, sample_weighted_kernel<IdT>, grid, SAMPLE_BLOCK, s, indices, probs,
                              static_cast<const IdT*>(seeds), n, k, replace, pv.row_begin, pv.deg, pv.local_off,
                              pv.tile_off, key, static_cast<IdT*>(coo_row), static_cast<IdT*>(coo_col), cap,
                              pos, rowpos, status));
  return DGS_OK;
}

}  // namespace

int64_t* sample_plan_total(void* plan, int64_t n_bound) { return plan_view(plan, n_bound).total; }
unsigned int* sample_plan_ticket(void* plan, int64_t n_bound) { return plan_view(plan, n_bound).ticket; }

uint64_t sample_rng_key(uint64_t rng_seed, uint64_t rng_offset) {
  return fold_rng_key(rng_seed, rng_offset);
}

int launch_sample_plan(const dgs_chunk_desc& indptr, const void* seeds, bool ids64, Count n, int64_t k,
                       bool replace, void* plan, int64_t* nnz_out, bool zero_ticket, const ClearJob& clear,
                       const LookupJob& lookup, int32_t* status, cudaStream_t s) {
  static_assert(SAMPLE_BLOCK == RL_BLOCK, "the jobs riding on the plan launch assume its CTA size");
  const PlanView pv = plan_view(plan, n.bound);
  if (zero_ticket) DGS_CUDA_TRY(cudaMemsetAsync(pv.ticket, 0, sizeof(unsigned int), s));
  return ids64 ? plan_typed<int64_t>(indptr, seeds, n, k, replace, pv, nnz_out, clear, lookup, status, s)
               : plan_typed<int32_t>(indptr, seeds, n, k, replace, pv, nnz_out, clear, lookup, status, s);
}

int launch_sample_uniform(const dgs_chunk_desc& indices, const void* seeds, bool ids64, Count n, int64_t k,
                          bool replace, void* plan, RngKey key, void* coo_row,
                          void* coo_col, int64_t out_capacity, int64_t* picked_pos, bool row_is_position,
                          int32_t* status, cudaStream_t s) {
  const PlanView pv = plan_view(plan, n.bound);
  return ids64 ? uniform_typed<int64_t>(indices, seeds, n, k, replace, pv, key, coo_row, coo_col,
                                        out_capacity, picked_pos, row_is_position, status, s)
               : uniform_typed<int32_t>(indices, seeds, n, k, replace, pv, key, coo_row, coo_col,
                                        out_capacity, picked_pos, row_is_position, status, s);
}

int launch_sample_weighted(const dgs_chunk_desc& indices, const dgs_chunk_desc& probs, const void* seeds,
                           bool ids64, Count n, int64_t k, bool replace, void* plan,
                           RngKey key, void* coo_row, void* coo_col, int64_t out_capacity,
                           int64_t* picked_pos, bool row_is_position, int32_t* status, cudaStream_t s) {
  const PlanView pv = plan_view(plan, n.bound);
  return ids64 ? weighted_typed<int64_t>(indices, probs, seeds, n, k, replace, pv, key, coo_row, coo_col,
                                         out_capacity, picked_pos, row_is_position, status, s)
               : weighted_typed<int32_t>(indices, probs, seeds, n, k, replace, pv, key, coo_row, coo_col,
                                         out_capacity, picked_pos, row_is_position, status, s);
}

}  // namespace dgs

extern "C" size_t dgs_sample_plan_bytes(int64_t n) {
  if (n < 0) n = 0;
  const int64_t ntiles = (n + dgs::SAMPLE_TILE - 1) / dgs::SAMPLE_TILE;
  return static_cast<size_t>(3 * n + ntiles + 2) * sizeof(int64_t);
}

extern "C" int dgs_sample_plan(const dgs_chunk_desc* indptr, const void* seeds, int32_t ids64,
                               int64_t n, int64_t k, int32_t replace, void* plan, int64_t* nnz,
                               int32_t* status, dgs_stream_t stream) {
  using namespace dgs;
  int rc = validate_desc(indptr, "dgs_sample_plan");
  if (rc != DGS_OK) return rc;
  rc = check_sample_args("dgs_sample_plan", seeds, n, k, plan);
  if (rc != DGS_OK) return rc;
  DGS_REQUIRE(indptr->esz == (ids64 ? 8 : 4), DGS_ERR_INVALID,
              "dgs_sample_plan: indptr element size %d does not match the id type", indptr->esz);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    if (nnz != nullptr) {
      zero_total_kernel<<<1, 1, 0, s>>>(nnz);
      DGS_LAUNCH_CHECK();
    }
    return DGS_OK;
  }
  return launch_sample_plan(*indptr, seeds, ids64 != 0, exact_count(n), k, replace != 0, plan, nnz, true, ClearJob{},
                            LookupJob{}, status, s);
}

extern "C" int dgs_sample_uniform(const dgs_chunk_desc* indices, const void* seeds, int32_t ids64,
                                  int64_t n, int64_t k, int32_t replace, const void* plan,
                                  uint64_t rng_seed, uint64_t rng_offset,
                                  void* coo_row, void* coo_col, int64_t out_capacity, int64_t* nnz,
                                  int64_t* picked_pos, int32_t* status, dgs_stream_t stream) {
  using namespace dgs;
  int rc = validate_desc(indices, "dgs_sample_uniform");
  if (rc != DGS_OK) return rc;
  rc = check_sample_args("dgs_sample_uniform", seeds, n, k, plan);
  if (rc != DGS_OK) return rc;
  DGS_REQUIRE(indices->esz == (ids64 ? 8 : 4), DGS_ERR_INVALID,
              "dgs_sample_uniform: indices element size %d does not match the id type", indices->esz);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n == 0 || k == 0) {
    if (nnz != nullptr) {
      zero_total_kernel<<<1, 1, 0, s>>>(nnz);
      DGS_LAUNCH_CHECK();
    }
    return DGS_OK;
  }
  DGS_REQUIRE(out_capacity == 0 || (coo_row != nullptr && coo_col != nullptr), DGS_ERR_INVALID,
              "dgs_sample_uniform: null output");
  rc = launch_sample_uniform(*indices, seeds, ids64 != 0, exact_count(n), k, replace != 0, const_cast<void*>(plan),
                             host_key(sample_rng_key(rng_seed, rng_offset)), coo_row, coo_col, out_capacity,
                             picked_pos, false, status, s);
  if (rc != DGS_OK) return rc;
  if (nnz != nullptr) {
    copy_total_kernel<<<1, 1, 0, s>>>(sample_plan_total(const_cast<void*>(plan), n), nnz);
    DGS_LAUNCH_CHECK();
  }
  return DGS_OK;
}

extern "C" int dgs_sample_weighted(const dgs_chunk_desc* indices, const dgs_chunk_desc* probs,
                                   const void* seeds, int32_t ids64, int64_t n, int64_t k,
                                   int32_t replace, const void* plan,
                                   uint64_t rng_seed, uint64_t rng_offset, void* coo_row, void* coo_col,
                                   int64_t out_capacity, int64_t* nnz, int64_t* picked_pos,
                                   int32_t* status, dgs_stream_t stream) {
  using namespace dgs;
  int rc = validate_desc(indices, "dgs_sample_weighted");
  if (rc != DGS_OK) return rc;
  rc = validate_desc(probs, "dgs_sample_weighted(probs)");
  if (rc != DGS_OK) return rc;
  rc = check_sample_args("dgs_sample_weighted", seeds, n, k, plan);
  if (rc != DGS_OK) return rc;
  DGS_REQUIRE(indices->esz == (ids64 ? 8 : 4), DGS_ERR_INVALID,
              "dgs_sample_weighted: indices element size %d does not match the id type", indices->esz);
  DGS_REQUIRE(probs->esz == 4, DGS_ERR_UNSUPPORTED, "dgs_sample_weighted: weights must be fp32");
  // the reference asserts the same bound on the device (rowwise_sampling_probs.cu:65)
  DGS_REQUIRE(replace || k <= 32, DGS_ERR_UNSUPPORTED,
              "dgs_sample_weighted: k=%lld > 32 without replacement is not supported", (long long)k);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n == 0 || k == 0) {
    if (nnz != nullptr) {
      zero_total_kernel<<<1, 1, 0, s>>>(nnz);
      DGS_LAUNCH_CHECK();
    }
    return DGS_OK;
  }
  DGS_REQUIRE(out_capacity == 0 || (coo_row != nullptr && coo_col != nullptr), DGS_ERR_INVALID,
              "dgs_sample_weighted: null output");
  rc = launch_sample_weighted(*indices, *probs, seeds, ids64 != 0, exact_count(n), k, replace != 0,
                              const_cast<void*>(plan), host_key(sample_rng_key(rng_seed, rng_offset)), coo_row,
                              coo_col, out_capacity, picked_pos, false, status, s);
  if (rc != DGS_OK) return rc;
  if (nnz != nullptr) {
    copy_total_kernel<<<1, 1, 0, s>>>(sample_plan_total(const_cast<void*>(plan), n), nnz);
    DGS_LAUNCH_CHECK();
  }
  return DGS_OK;
}
