// Exclusive scan of per-tile sums: the middle step of every "count per tile ->
// scan tile sums -> write with known offsets" sequence in this library (sample
// offsets, first-occurrence numbering, split-index classes).  Replaces the
// reference's cub::DeviceScan wrapper (src/cuda/cub_function.h:10-22) plus its
// blocking read-back of the last element (src/cuda/rowwise_sampling.cu:147,
// src/cuda/tensor_reindex.cu:129): the totals go straight to a caller-supplied
// (normally pinned) location, so the host reads them whenever it next
// synchronises instead of stalling mid-sequence.
#pragma once
#include "common.cuh"

namespace dgs {

constexpr int TILE_SCAN_BLOCK = 1024;

// sums: [ntiles][C] tile-major.  In place: sums[t][c] becomes the exclusive
// prefix over tiles; totals_dev[c] (device scratch, optional) and
// totals_out[c] (optional) receive the grand totals.  One CTA.
template <int C>
__global__ void __launch_bounds__(TILE_SCAN_BLOCK)
tile_scan_kernel(int64_t* __restrict__ sums, const int64_t ntiles, int64_t* __restrict__ totals_dev,
                 int64_t* __restrict__ totals_out) {
  __shared__ int64_t smem[TILE_SCAN_BLOCK / 32 + 1];
  int64_t carry[C];
#pragma unroll
  for (int c = 0; c < C; ++c) carry[c] = 0;
  for (int64_t t0 = 0; t0 < ntiles; t0 += TILE_SCAN_BLOCK) {
    const int64_t t = t0 + threadIdx.x;
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const int64_t v = (t < ntiles) ? sums[t * C + c] : 0;
      int64_t total;
      const int64_t ex = block_exclusive_scan<int64_t, TILE_SCAN_BLOCK>(v, smem, &total);
      if (t < ntiles) sums[t * C + c] = carry[c] + ex;
      carry[c] += total;
    }
  }
  if (threadIdx.x == 0) {
#pragma unroll
    for (int c = 0; c < C; ++c) {
      if (totals_dev != nullptr) totals_dev[c] = carry[c];
      if (totals_out != nullptr) totals_out[c] = carry[c];
    }
  }
}


// The same scan without a second launch: every CTA of a counting kernel calls
// this after computing its tile sum.  The CTA that draws the last ticket (an
// atomic counter that must be zero at launch; nobody waits on anybody) scans
// all tile sums in place and publishes the total.  `smem` needs BLOCK/32 + 1
// entries; must be called by all threads of the CTA.  Returns true in that last CTA.
// The tiles are CTAs 0 .. ntiles-1 of the launch (the launch may hold further CTAs
// with other work, which do not call this).
template <int BLOCK>
__device__ __forceinline__ bool publish_and_scan_tiles(int64_t my_tile_sum, int64_t* tile_sums,
                                                       unsigned int* ticket, int64_t* total_dev,
                                                       int64_t* total_out, int64_t* smem,
                                                       unsigned int n_tiles = 0) {
  __shared__ bool s_last;
  if (n_tiles == 0) n_tiles = gridDim.x;
  if (threadIdx.x == 0) {
    tile_sums[blockIdx.x] = my_tile_sum;
    __threadfence();
    s_last = atomicAdd(ticket, 1u) == n_tiles - 1;
  }
  __syncthreads();
  if (!s_last) return false;
  __threadfence();
  // Every thread takes a contiguous run of `per` tiles: all loads of the CTA are issued together (one round
  // trip to L2 whatever the number of tiles, instead of one per BLOCK tiles), one block scan over the threads'
  // sums gives each run its offset, and a second walk over the run (now in L1/L2) writes the prefixes.  This
  // CTA works alone at the end of its kernel, so every microsecond here is latency of the whole sequence.
  const int64_t ntiles = n_tiles;
  const int64_t per = (ntiles + BLOCK - 1) / BLOCK;
  const int64_t lo = static_cast<int64_t>(threadIdx.x) * per;
  const int64_t hi = lo + per < ntiles ? lo + per : ntiles;
  int64_t mine = 0;
  for (int64_t t = lo; t < hi; ++t) mine += __ldcg(tile_sums + t);
  int64_t carry;
  int64_t run = block_exclusive_scan<int64_t, BLOCK>(mine, smem, &carry);
  for (int64_t t = lo; t < hi; ++t) {
    const int64_t v = __ldcg(tile_sums + t);
    tile_sums[t] = run;
    run += v;
  }
  if (threadIdx.x == 0) {
    if (total_dev != nullptr) *total_dev = carry;
    *ticket = 0;
    if (total_out != nullptr) {
      *total_out = carry;
      __threadfence_system();
    }
  }
  return true;  // this CTA was the last one: the totals are final
}

}  // namespace dgs
