// Split row ids by location class (local chunk / peer chunks / host tail).
//
// Replaces _GetSplitIndexMaskKernel and the three boolean-mask selects that
// follow it (reference src/cuda/index_with_chunk_tensor.cu:55-108): there, a
// 128-thread block per id writes three bool masks (every thread of the block
// doing the same work) and torch's mask-select runs three nonzero+gather
// passes, each with its own host synchronisation.
//
// Here it is one stable three-way partition: count per tile, scan the tile
// sums, scatter.  The class predicates are the reference's integer divisions,
// evaluated once on the host:
//   host   : id >= threshold / D
//   local  : rank*each / D <= id < (rank+1)*each / D
//   remote : everything else
// Output is one array [local ids | remote ids | host ids], each class in input
// order, and the three class sizes.
#include <mutex>

#include "common.cuh"
#include "tile_scan.cuh"

namespace dgs {
namespace {

constexpr int SPLIT_BLOCK = 256;
constexpr int SPLIT_ITEMS = 8;
constexpr int SPLIT_TILE = SPLIT_BLOCK * SPLIT_ITEMS;

struct SplitBounds {
  int64_t host_lo, loc_lo, loc_hi;
};

__device__ __forceinline__ int classify(int64_t r, const SplitBounds& b) {
  if (r >= b.host_lo) return 2;
  if (r >= b.loc_lo && r < b.loc_hi) return 0;
  return 1;
}

template <typename IdxT>
__global__ void __launch_bounds__(SPLIT_BLOCK)
split_count_kernel(const IdxT* __restrict__ idx, const int64_t n, const SplitBounds b,
                   int64_t* __restrict__ tile_counts) {
  __shared__ unsigned long long s_acc;
  if (threadIdx.x == 0) s_acc = 0ull;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * SPLIT_TILE + threadIdx.x * SPLIT_ITEMS;
  unsigned long long packed = 0ull;
#pragma unroll
  for (int u = 0; u < SPLIT_ITEMS; ++u) {
    const int64_t i = base + u;
    if (i < n) packed += 1ull << (21 * classify(static_cast<int64_t>(idx[i]), b));
  }
  // warp reduce, then one shared atomic per warp
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) packed += __shfl_down_sync(FULL_MASK, packed, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(&s_acc, packed);
  __syncthreads();
  if (threadIdx.x < 3)
    tile_counts[static_cast<int64_t>(blockIdx.x) * 3 + threadIdx.x] =
        static_cast<int64_t>((s_acc >> (21 * threadIdx.x)) & 0x1FFFFFull);
}

template <typename IdxT>
__global__ void __launch_bounds__(SPLIT_BLOCK)
split_scatter_kernel(const IdxT* __restrict__ idx, const int64_t n, const SplitBounds b,
                     const int64_t* __restrict__ tile_offsets, const int64_t* __restrict__ totals,
                     IdxT* __restrict__ out) {
  __shared__ unsigned long long smem[SPLIT_BLOCK / 32 + 1];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * SPLIT_TILE + threadIdx.x * SPLIT_ITEMS;
  IdxT v[SPLIT_ITEMS];
  int cls[SPLIT_ITEMS];
  unsigned long long packed = 0ull;
#pragma unroll
  for (int u = 0; u < SPLIT_ITEMS; ++u) {
    const int64_t i = base + u;
    cls[u] = -1;
    if (i < n) {
      v[u] = idx[i];
      cls[u] = classify(static_cast<int64_t>(v[u]), b);
      packed += 1ull << (21 * cls[u]);
    }
  }
  unsigned long long total;
  const unsigned long long ex =
      block_exclusive_scan<unsigned long long, SPLIT_BLOCK>(packed, smem, &total);
  int64_t pos[3];
  const int64_t class_base[3] = {0, totals[0], totals[0] + totals[1]};
#pragma unroll
  for (int c = 0; c < 3; ++c)
    pos[c] = class_base[c] + tile_offsets[static_cast<int64_t>(blockIdx.x) * 3 + c] +
             static_cast<int64_t>((ex >> (21 * c)) & 0x1FFFFFull);
#pragma unroll
  for (int u = 0; u < SPLIT_ITEMS; ++u) {
    if (cls[u] == 0) out[pos[0]++] = v[u];
    else if (cls[u] == 1) out[pos[1]++] = v[u];
    else if (cls[u] == 2) out[pos[2]++] = v[u];
  }
}

template <typename IdxT>
int run_split(const void* idx, int64_t n, const SplitBounds& b, void* out, int64_t* counts,
              int64_t* scratch, cudaStream_t stream) {
  const int64_t ntiles = (n + SPLIT_TILE - 1) / SPLIT_TILE;
  int64_t* tile_counts = scratch;          // [ntiles][3]
  int64_t* totals = scratch + ntiles * 3;  // [3]
  split_count_kernel<IdxT><<<static_cast<unsigned>(ntiles), SPLIT_BLOCK, 0, stream>>>(
      static_cast<const IdxT*>(idx), n, b, tile_counts);
  DGS_LAUNCH_CHECK();
  tile_scan_kernel<3><<<1, TILE_SCAN_BLOCK, 0, stream>>>(tile_counts, ntiles, totals, counts);
  DGS_LAUNCH_CHECK();
  split_scatter_kernel<IdxT><<<static_cast<unsigned>(ntiles), SPLIT_BLOCK, 0, stream>>>(
      static_cast<const IdxT*>(idx), n, b, tile_counts, totals, static_cast<IdxT*>(out));
  DGS_LAUNCH_CHECK();
  return DGS_OK;
}

__global__ void zero_counts_kernel(int64_t* counts) {
  if (threadIdx.x < 3) counts[threadIdx.x] = 0;
}

// ---- scratch for dgs_split_index_static ---------------------------------------
// Lives in the library image: every GPU that loads the library holds these
// 192 KB until the process exits.  Layout as in run_split: [tiles][3] counts,
// then 3 totals.
constexpr int64_t SPLIT_STATIC_WORDS = (DGS_SPLIT_STATIC_MAX_IDS / SPLIT_TILE) * 3 + 3;
static __device__ __align__(256) int64_t g_split_static[SPLIT_STATIC_WORDS];

// In host code `g_split_static` is only a handle for the runtime, not an
// address a kernel may use; the device address is looked up once per device,
// with that device current.
int split_static_scratch(int64_t** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int64_t* addr[kMaxDevices] = {};
  int dev = -1;
  DGS_CUDA_TRY(cudaGetDevice(&dev));
  DGS_REQUIRE(dev >= 0 && dev < kMaxDevices, DGS_ERR_UNSUPPORTED, "device index %d is not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    DGS_CUDA_TRY(cudaGetSymbolAddress(&p, g_split_static));
    DGS_REQUIRE(p != nullptr, DGS_ERR_CUDA, "no device address for the static split scratch");
    addr[dev] = static_cast<int64_t*>(p);
  }
  *out = addr[dev];
  return DGS_OK;
}

}  // namespace
}  // namespace dgs

extern "C" size_t dgs_split_index_scratch_bytes(int64_t n) {
  if (n < 0) n = 0;
  const int64_t ntiles = (n + dgs::SPLIT_TILE - 1) / dgs::SPLIT_TILE;
  return static_cast<size_t>(ntiles * 3 + 3) * sizeof(int64_t);
}

extern "C" int dgs_split_index(const dgs_chunk_desc* t, const void* idx, int32_t ids64, int64_t n,
                               int64_t D, void* out, int64_t* counts, void* scratch,
                               size_t scratch_bytes, dgs_stream_t stream) {
  using namespace dgs;
  int rc = validate_desc(t, "dgs_split_index");
  if (rc != DGS_OK) return rc;
  DGS_REQUIRE(n >= 0 && D >= 1 && counts != nullptr, DGS_ERR_INVALID, "dgs_split_index: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    zero_counts_kernel<<<1, 32, 0, s>>>(counts);
    DGS_LAUNCH_CHECK();
    return DGS_OK;
  }
  DGS_REQUIRE(idx != nullptr && out != nullptr && scratch != nullptr, DGS_ERR_INVALID,
              "dgs_split_index: null buffer");
  DGS_REQUIRE(scratch_bytes >= dgs_split_index_scratch_bytes(n), DGS_ERR_INVALID,
              "dgs_split_index: scratch too small");
  DGS_REQUIRE((n + SPLIT_TILE - 1) / SPLIT_TILE <= 0x7fffffffLL, DGS_ERR_UNSUPPORTED,
              "dgs_split_index: too many ids");
  SplitBounds b;
  b.host_lo = t->threshold / D;
  b.loc_lo = static_cast<int64_t>(t->local_rank) * t->each / D;
  b.loc_hi = static_cast<int64_t>(t->local_rank + 1) * t->each / D;
  return ids64 ? run_split<int64_t>(idx, n, b, out, counts, static_cast<int64_t*>(scratch), s)
               : run_split<int32_t>(idx, n, b, out, counts, static_cast<int64_t*>(scratch), s);
}

extern "C" int dgs_split_index_static(const dgs_chunk_desc* t, const void* idx, int32_t ids64, int64_t n,
                                      int64_t D, void* out, int64_t* counts, dgs_stream_t stream) {
  using namespace dgs;
  int rc = validate_desc(t, "dgs_split_index_static");
  if (rc != DGS_OK) return rc;
  DGS_REQUIRE(n >= 0 && D >= 1 && counts != nullptr, DGS_ERR_INVALID, "dgs_split_index_static: bad arguments");
  DGS_REQUIRE(n <= DGS_SPLIT_STATIC_MAX_IDS, DGS_ERR_UNSUPPORTED,
              "dgs_split_index_static: %lld ids exceed the built-in scratch (at most %lld per call); "
              "use dgs_split_index with caller-provided scratch",
              (long long)n, (long long)DGS_SPLIT_STATIC_MAX_IDS);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    zero_counts_kernel<<<1, 32, 0, s>>>(counts);
    DGS_LAUNCH_CHECK();
    return DGS_OK;
  }
  DGS_REQUIRE(idx != nullptr && out != nullptr, DGS_ERR_INVALID, "dgs_split_index_static: null buffer");
  int64_t* scratch = nullptr;
  rc = split_static_scratch(&scratch);  // first call on a device: looks the address up
  if (rc != DGS_OK) return rc;
  SplitBounds b;
  b.host_lo = t->threshold / D;
  b.loc_lo = static_cast<int64_t>(t->local_rank) * t->each / D;
  b.loc_hi = static_cast<int64_t>(t->local_rank + 1) * t->each / D;
  // every scratch word a call reads (tile counts, totals) is written earlier in
  // the same call, so nothing left over from the previous call needs clearing
  return ids64 ? run_split<int64_t>(idx, n, b, out, counts, scratch, s)
               : run_split<int32_t>(idx, n, b, out, counts, scratch, s);
}
