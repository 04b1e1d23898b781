// Locality order: a permutation of the request that visits ids in (coarse)
// address order.
//
// An optional tool, off by default.  It pays when address translation, not
// bandwidth, limits a request: with a peer mapping that had ended up on small
// pages (a chunk whose size was not a multiple of 2 MB, see store.cc), random
// 512-byte rows over a 25 GB peer range ran at 105 GB/s unordered and 590 GB/s
// ordered on B200.  With chunks padded to 2 MB the same request runs at
// 635 GB/s unordered and ordering costs ~6 %, so the operator layer only uses
// it when DGS_LOCALITY_ORDER=1.  The kernels take the permutation as an
// optional argument and still write every result to the place its id has in
// the request, so the output is unchanged.
//
// The order is a counting sort on the high bits of the id (4096 bins; ids
// within a bin stay unordered): histogram, one-CTA scan, scatter.
#include "common.cuh"

namespace dgs {
namespace {

constexpr int ORDER_BINS_LOG2 = 12;
constexpr int ORDER_BINS = 1 << ORDER_BINS_LOG2;
constexpr int ORDER_BLOCK = 512;
constexpr int ORDER_ITEMS = 8;

template <typename IdT>
__device__ __forceinline__ uint32_t bin_of(IdT id, int shift) {
  if (id < 0) return 0;
  const uint64_t b = static_cast<uint64_t>(id) >> shift;
  return b < ORDER_BINS ? static_cast<uint32_t>(b) : ORDER_BINS - 1;
}

template <typename IdT>
__global__ void __launch_bounds__(ORDER_BLOCK)
order_hist_kernel(const IdT* __restrict__ ids, const int64_t n, const int shift, uint32_t* __restrict__ counts) {
  __shared__ uint32_t s_hist[ORDER_BINS];
  for (int b = threadIdx.x; b < ORDER_BINS; b += ORDER_BLOCK) s_hist[b] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (ORDER_BLOCK * ORDER_ITEMS) + threadIdx.x;
#pragma unroll
  for (int u = 0; u < ORDER_ITEMS; ++u) {
    const int64_t i = base + static_cast<int64_t>(u) * ORDER_BLOCK;
    if (i < n) atomicAdd(&s_hist[bin_of(ids[i], shift)], 1u);
  }
  __syncthreads();
  for (int b = threadIdx.x; b < ORDER_BINS; b += ORDER_BLOCK) {
    const uint32_t c = s_hist[b];
    if (c) atomicAdd(&counts[b], c);
  }
}

// counts[bins] -> cursor[bins] = exclusive prefix (one CTA, 4 bins per thread)
__global__ void __launch_bounds__(1024) order_scan_kernel(const uint32_t* __restrict__ counts,
                                                          uint32_t* __restrict__ cursor) {
  __shared__ uint32_t smem[1024 / 32 + 1];
  constexpr int PER = ORDER_BINS / 1024;
  uint32_t v[PER], sum = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    v[j] = counts[threadIdx.x * PER + j];
    sum += v[j];
  }
  uint32_t total;
  uint32_t ex = block_exclusive_scan<uint32_t, 1024>(sum, smem, &total);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    cursor[threadIdx.x * PER + j] = ex;
    ex += v[j];
  }
}

template <typename IdT>
__global__ void __launch_bounds__(ORDER_BLOCK)
order_scatter_kernel(const IdT* __restrict__ ids, const int64_t n, const int shift, uint32_t* cursor,
                     uint32_t* __restrict__ order) {
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (ORDER_BLOCK * ORDER_ITEMS) + threadIdx.x;
#pragma unroll
  for (int u = 0; u < ORDER_ITEMS; ++u) {
    const int64_t i = base + static_cast<int64_t>(u) * ORDER_BLOCK;
    if (i < n) order[atomicAdd(&cursor[bin_of(ids[i], shift)], 1u)] = static_cast<uint32_t>(i);
  }
}

template <typename IdT>
int run_order(const void* ids, int64_t n, int shift, uint32_t* order, uint32_t* counts, uint32_t* cursor,
              cudaStream_t s) {
  const unsigned grid = static_cast<unsigned>((n + ORDER_BLOCK * ORDER_ITEMS - 1) / (ORDER_BLOCK * ORDER_ITEMS));
  DGS_CUDA_TRY(cudaMemsetAsync(counts, 0, ORDER_BINS * sizeof(uint32_t), s));
  order_hist_kernel<IdT><<<grid, ORDER_BLOCK, 0, s>>>(static_cast<const IdT*>(ids), n, shift, counts);
  DGS_LAUNCH_CHECK();
  order_scan_kernel<<<1, 1024, 0, s>>>(counts, cursor);
  DGS_LAUNCH_CHECK();
  order_scatter_kernel<IdT><<<grid, ORDER_BLOCK, 0, s>>>(static_cast<const IdT*>(ids), n, shift, cursor, order);
  DGS_LAUNCH_CHECK();
  return DGS_OK;
}

}  // namespace
}  // namespace dgs

extern "C" size_t dgs_locality_order_scratch_bytes(void) { return 2 * dgs::ORDER_BINS * sizeof(uint32_t); }

extern "C" int dgs_locality_order(const void* ids, int32_t ids64, int64_t n, int64_t id_space, uint32_t* order,
                                  void* scratch, size_t scratch_bytes, dgs_stream_t stream) {
  using namespace dgs;
  DGS_REQUIRE(n >= 0 && n <= 0xFFFFFFFFll && id_space >= 1, DGS_ERR_INVALID,
              "dgs_locality_order: n=%lld id_space=%lld", (long long)n, (long long)id_space);
  if (n == 0) return DGS_OK;
  DGS_REQUIRE(ids != nullptr && order != nullptr && scratch != nullptr &&
                  scratch_bytes >= dgs_locality_order_scratch_bytes(),
              DGS_ERR_INVALID, "dgs_locality_order: null buffer or scratch too small");
  int bits = 0;
  while (bits < 63 && (int64_t(1) << bits) < id_space) ++bits;
  const int shift = bits > ORDER_BINS_LOG2 ? bits - ORDER_BINS_LOG2 : 0;
  uint32_t* counts = static_cast<uint32_t*>(scratch);
  uint32_t* cursor = counts + ORDER_BINS;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ids64 ? run_order<int64_t>(ids, n, shift, order, counts, cursor, s)
               : run_order<int32_t>(ids, n, shift, order, counts, cursor, s);
}
