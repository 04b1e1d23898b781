// Row gather over a ChunkTensor:  out[i, :] = T[idx[i], :]
//
// Replaces _IndexMemcpyKernel / _Local.. / _Remote.. / _HostIndexMemcpyKernel
// (reference src/cuda/index_with_chunk_tensor.cu:9-27,110-168), which run one
// 128-thread block per row with scalar 4/8-byte accesses and re-resolve the
// owner (three dependent metadata loads + a 64-bit divide) for every element.
//
// Design (HBM-bound copy, no tensor cores):
//   * a CTA owns a tile of R consecutive output rows.  Phase 1 resolves each
//     row ONCE (owner chunk / host tail, bounds, straddle) and parks the source
//     pointer in shared memory.  Phase 2 treats the tile as R*nvec vectors of
//     VEC bytes: consecutive threads move consecutive 16-byte pieces, so every
//     lane is busy whatever the row width (D = 100 fp32 -> 25 vectors/row) and
//     the output side is one contiguous, fully coalesced stream.  Eight
//     independent vector loads are in flight per thread before the first store.
//   * VEC (16/8/4/2/1 bytes) is picked on the host as the largest power of two
//     dividing the row size and every base offset, so all rows that lie inside
//     one storage region take the vector path.  Rows that straddle a chunk
//     boundary (at most one per boundary in the whole tensor) and out-of-range
//     ids take a per-element path; out-of-range rows are zero-filled and
//     reported through the status word instead of faulting.
//   * peer chunks (cudaIpc-mapped, NVLink) and the host tail (pinned, UVA) are
//     ordinary global addresses, read with the same ld.global.nc vector loads.
#include <atomic>
#include <cstdlib>

#include "common.cuh"

namespace dgs {
namespace {

constexpr int GATHER_BLOCK = 256;
constexpr int GATHER_UNROLL = 8;
constexpr int GATHER_MAX_ROWS = 1024;  // rows per tile upper bound (smem: 8 KB)

template <int VEC> struct VecT;
template <> struct VecT<16> { using type = uint4; };
template <> struct VecT<8> { using type = uint2; };
template <> struct VecT<4> { using type = uint32_t; };
template <> struct VecT<2> { using type = uint16_t; };
template <> struct VecT<1> { using type = uint8_t; };

// tags stored in the shared pointer table
#define DGS_ROW_ZERO reinterpret_cast<const char*>(uintptr_t(0))
#define DGS_ROW_SLOW reinterpret_cast<const char*>(uintptr_t(1))

// ---- rows that do not start on a vector boundary --------------------------------
// A capacity_per_gpu that is not a multiple of the row size puts every row of the later chunks and of
// the host tail at an odd offset.  Such a row is still read with aligned vector loads: output vector j is
// cut out of the aligned vectors A_j and A_j+1 that cover it (A_j+1 comes from the lane to the right, or
// from one more load at the row's end), so the row costs the same requests as an aligned one.  Needs
// 4-byte elements at least (the offset is then a whole number of words) and room for the last aligned
// vector, which reaches up to VEC - 4 bytes past the row, inside the row's storage region.
template <int VEC, bool REALIGN>
__device__ __forceinline__ bool vector_copy_ok(const char* src, int64_t run_bytes, int64_t row_bytes) {
  const uintptr_t mis = reinterpret_cast<uintptr_t>(src) & (VEC - 1);
  if (mis == 0) return true;
  return REALIGN && (mis & 3) == 0 && run_bytes >= row_bytes + VEC - static_cast<int64_t>(mis);
}
__device__ __forceinline__ uint4 cut_vector(const uint4& a, const uint4& b, uint32_t words) {
  switch (words) {
    case 1: return make_uint4(a.y, a.z, a.w, b.x);
    case 2: return make_uint4(a.z, a.w, b.x, b.y);
    case 3: return make_uint4(a.w, b.x, b.y, b.z);
    default: return a;
  }
}
__device__ __forceinline__ uint2 cut_vector(const uint2& a, const uint2& b, uint32_t words) {
  return words ? make_uint2(a.y, b.x) : a;
}
template <typename V>
__device__ __forceinline__ V cut_vector(const V& a, const V&, uint32_t) { return a; }  // narrower: always aligned
__device__ __forceinline__ uint4 shfl_right(const uint4& v) {
  return make_uint4(__shfl_down_sync(FULL_MASK, v.x, 1), __shfl_down_sync(FULL_MASK, v.y, 1),
                    __shfl_down_sync(FULL_MASK, v.z, 1), __shfl_down_sync(FULL_MASK, v.w, 1));
}
__device__ __forceinline__ uint2 shfl_right(const uint2& v) {
  return make_uint2(__shfl_down_sync(FULL_MASK, v.x, 1), __shfl_down_sync(FULL_MASK, v.y, 1));
}
template <typename V>
__device__ __forceinline__ V shfl_right(const V& v) { return v; }

// ---- row sources ------------------------------------------------------------
// A row source maps output row i to the address of its D elements, or to one
// of the two tags above.  `slow_row` copies a tagged-slow row element-wise.

// rows of a ChunkTensor selected by idx[i]
template <typename IdxT>
struct ChunkRows {
  dgs_chunk_desc d;
  const IdxT* idx;
  int64_t D;
  int64_t n_rows_total;  // rows lying fully inside the tensor
  int sh;

  // the requested row id at position i, and where that row lives
  __device__ __forceinline__ int64_t row_id(int64_t i) const { return static_cast<int64_t>(idx[i]); }
  template <int VEC, bool REALIGN>
  __device__ __forceinline__ const char* locate(int64_t i, int32_t* status) const {
    return locate_row<VEC, REALIGN>(row_id(i), status);
  }
  template <int VEC, bool REALIGN>
  __device__ __forceinline__ const char* locate_row(int64_t row, int32_t* status) const {
    if (row < 0 || row >= n_rows_total) {
      raise_status(status, DGS_ERR_RANGE);
      return DGS_ROW_ZERO;
    }
    int64_t run;
    const char* src = resolve(d, sh, row * D, &run);
    if (run < D || !vector_copy_ok<VEC, REALIGN>(src, run << sh, D << sh)) return DGS_ROW_SLOW;
    return src;
  }
  __device__ __forceinline__ const char* element(int64_t i, int64_t j) const {
    int64_t run;
    return resolve(d, sh, static_cast<int64_t>(idx[i]) * D + j, &run);
  }
};

// PaGraph-style cached rows: nid[i] is looked up in an open-addressing table
// (keys/values); a hit reads row `value` of the GPU-side ChunkTensor, a miss
// reads row nid[i] of the device-visible host array.
// Replaces _FetchDataKernel / _FetchDataWithChunkTensorKernel
// (reference src/cuda/pagraph.cu:126-194).
__device__ __forceinline__ uint64_t cache_hash(long long key) {
  uint64_t z = static_cast<uint64_t>(key);
  z = (z ^ (z >> 33)) * 0xFF51AFD7ED558CCDull;
  z = (z ^ (z >> 33)) * 0xC4CEB9FE1A85EC53ull;
  return z ^ (z >> 33);
}

template <typename IdxT>
struct CachedRows {
  dgs_chunk_desc gpu;
  const char* cpu_data;
  const IdxT* nid;
  const IdxT* keys;
  const IdxT* values;
  uint64_t mask;  // slots - 1
  int64_t D;
  int64_t gpu_rows;
  int64_t cpu_rows;
  int sh;

  __device__ __forceinline__ int64_t cached_row(int64_t id) const {
    uint64_t h = cache_hash(id) & mask;
    for (uint64_t probes = 0; probes <= mask; ++probes) {
      const long long k = static_cast<long long>(keys[h]);
      if (k == id) return static_cast<int64_t>(values[h]);
      if (k == -1) return -1;
      h = (h + 1) & mask;
    }
    return -1;
  }
  template <int VEC, bool REALIGN>
  __device__ __forceinline__ const char* locate(int64_t i, int32_t* status) const {
    const int64_t id = static_cast<int64_t>(nid[i]);
    if (id < 0) {
      raise_status(status, DGS_ERR_RANGE);
      return DGS_ROW_ZERO;
    }
    const int64_t row = cached_row(id);
    if (row < 0 && id < cpu_rows) return cpu_data + (id * D << sh);  // miss: host row
    if (row < 0 || row >= gpu_rows) {
      raise_status(status, DGS_ERR_RANGE);
      return DGS_ROW_ZERO;
    }
    int64_t run;
    const char* src = resolve(gpu, sh, row * D, &run);
    if (run < D || !vector_copy_ok<VEC, REALIGN>(src, run << sh, D << sh)) return DGS_ROW_SLOW;
    return src;
  }
  __device__ __forceinline__ const char* element(int64_t i, int64_t j) const {
    int64_t run;  // only cached rows can be tagged slow
    return resolve(gpu, sh, cached_row(static_cast<int64_t>(nid[i])) * D + j, &run);
  }
};

template <typename Src, int VEC, bool REALIGN>
__global__ void __launch_bounds__(GATHER_BLOCK)
gather_rows_kernel(const __grid_constant__ Src rows, const int64_t n_bound, const int64_t* __restrict__ n_dev,
                   const int64_t D, const int sh, const uint32_t nvec, const uint32_t rows_per_tile, const uint32_t div_magic,
                   const uint32_t slot_shift,
                   char* __restrict__ out, int32_t* __restrict__ status) {
  using V = typename VecT<VEC>::type;
  __shared__ const char* s_src[GATHER_MAX_ROWS];
  pdl_enter();

  // the number of rows is the host's (n_dev == nullptr) or a device word written by an earlier kernel on
  // the stream, with n_bound the upper limit the grid was sized for: CTAs past the live count leave at once
  int64_t n = n_bound;
  if (n_dev != nullptr) {
    const int64_t live = *n_dev;
    n = live < n_bound ? (live < 0 ? 0 : live) : n_bound;
  }
  const int64_t tile_row0 = static_cast<int64_t>(blockIdx.x) * rows_per_tile;
  if (tile_row0 >= n) return;
  const uint32_t rows_here =
      static_cast<uint32_t>(min(static_cast<int64_t>(rows_per_tile), n - tile_row0));

  // ---- phase 1: one resolution per row -------------------------------------
  bool any_special = false;
  for (uint32_t r = threadIdx.x; r < rows_here; r += GATHER_BLOCK) {
    const char* src = rows.template locate<VEC, REALIGN>(tile_row0 + r, status);
    any_special |= (reinterpret_cast<uintptr_t>(src) <= 1);
    s_src[r] = src;
  }
  const int block_special = __syncthreads_or(any_special ? 1 : 0);

  // ---- phase 2: vector copy, contiguous on the output side -----------------
  // Item q of the tile is vector j of row r.  Flat mode (slot_shift == 0): q = r * nvec + j, every lane
  // busy, a warp's load may end one row and begin the next.  Slot mode: every row owns 2^slot_shift lanes
  // (the power of two >= nvec), so one warp-wide load never splits a row between two instructions; the
  // lanes past the row's end idle.  Fewer, fuller requests is what a peer or host link wants.
  const uint32_t items = slot_shift ? (rows_here << slot_shift) : rows_here * nvec;
  V* __restrict__ out_tile = reinterpret_cast<V*>(out + (tile_row0 * D << sh));
  constexpr int UNROLL = REALIGN ? GATHER_UNROLL / 2 : GATHER_UNROLL;  // loads in flight per thread
  for (uint32_t q0 = 0; q0 < items; q0 += GATHER_BLOCK * UNROLL) {
    V v[UNROLL];
    V tail[REALIGN ? UNROLL : 1];  // REALIGN: A_j+1 for the lanes that cannot get it from their neighbour
    uint32_t at[UNROLL];           // where the vector goes: row r, vector j; ~0u: nothing to store
    uint32_t cut = 0;              // REALIGN: 4 bits per u -- bit 3: own tail load, bits 0-1: offset in words
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const uint32_t q = q0 + u * GATHER_BLOCK + threadIdx.x;
      at[u] = ~0u;
      const char* src = nullptr;
      uint32_t j = 0;
      if (q < items) {
        uint32_t r;
        if (slot_shift) {
          r = q >> slot_shift;
          j = q & ((1u << slot_shift) - 1u);
        } else {
          // q / nvec, exact while q*nvec < 2^32 (div_magic = ceil(2^32 / nvec); 0: nvec == 1)
          r = rows_per_tile == 1 ? 0u : (div_magic ? __umulhi(q, div_magic) : q);
          j = q - r * nvec;
        }
        src = s_src[r];
        if (j < nvec && reinterpret_cast<uintptr_t>(src) > 1)
          at[u] = rows_per_tile == 1 ? j : ((r << 16) | j);  // several rows per tile: r < 1024, j < 2048
      }
      if (!REALIGN) {
        if (at[u] != ~0u) v[u] = ld_stream(reinterpret_cast<const V*>(src) + j);
      } else {
        // all 32 lanes come through here: the neighbour test is a shuffle
        const uint32_t mis = at[u] != ~0u ? static_cast<uint32_t>(reinterpret_cast<uintptr_t>(src) & (VEC - 1)) : 0u;
        const char* a0 = src - mis + static_cast<size_t>(j) * VEC;  // aligned vector that holds the row's vector j
        if (at[u] != ~0u) v[u] = ld_stream(reinterpret_cast<const V*>(a0));
        // the lane to the right holds A_j+1 iff it serves vector j + 1 of the same row
        const uint32_t right = __shfl_down_sync(FULL_MASK, at[u], 1);
        const bool from_right = (threadIdx.x & 31) != 31 && at[u] != ~0u && right == at[u] + 1;
        const bool own_tail = mis != 0 && !from_right;
        if (own_tail) tail[u] = ld_stream(reinterpret_cast<const V*>(a0 + VEC));
        cut |= ((mis >> 2) | (own_tail ? 8u : 0u)) << (4 * u);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (REALIGN) {
        const V next = shfl_right(v[u]);  // executed by all lanes
        const uint32_t c = (cut >> (4 * u)) & 15u;
        if (c & 7u) v[u] = cut_vector(v[u], (c & 8u) ? tail[u] : next, c & 7u);
      }
      if (at[u] != ~0u) {
        const uint32_t r = rows_per_tile == 1 ? 0u : (at[u] >> 16);
        const uint32_t j = rows_per_tile == 1 ? at[u] : (at[u] & 0xFFFFu);
        out_tile[r * nvec + j] = v[u];
      }
    }
  }

  // ---- phase 3: rare rows (straddle a chunk boundary / out of range) -------
  if (block_special) {
    const int esz = 1 << sh;
    for (uint32_t r = 0; r < rows_here; ++r) {
      const char* src = s_src[r];
      if (reinterpret_cast<uintptr_t>(src) > 1) continue;
      const int64_t i = tile_row0 + r;  // request position of this row
      char* dst = out + (i * D << sh);
      if (src == DGS_ROW_ZERO) {
        for (int64_t b = threadIdx.x; b < (D << sh); b += GATHER_BLOCK) dst[b] = 0;
      } else {
        for (int64_t j = threadIdx.x; j < D; j += GATHER_BLOCK) {
          const char* p = rows.element(i, j);
          char* q = dst + (j << sh);
          switch (esz) {
            case 8: *reinterpret_cast<uint64_t*>(q) = *reinterpret_cast<const uint64_t*>(p); break;
            case 4: *reinterpret_cast<uint32_t*>(q) = *reinterpret_cast<const uint32_t*>(p); break;
            case 2: *reinterpret_cast<uint16_t*>(q) = *reinterpret_cast<const uint16_t*>(p); break;
            default: *q = *p; break;
          }
        }
      }
    }
  }
}

template <typename Src, int VEC, bool REALIGN>
int launch_gather_r(const Src& rows, Count nc, int64_t D, int sh, void* out, int32_t* status,
                    cudaStream_t stream) {
  const int64_t n = nc.bound;
  const int64_t row_bytes = D << sh;
  const int64_t nvec64 = row_bytes / VEC;
  // the in-tile index q < rows*nvec must keep q*nvec < 2^32 for the magic divide
  DGS_REQUIRE(nvec64 <= (1 << 24), DGS_ERR_UNSUPPORTED, "gather: rows of %lld bytes are not supported",
              (long long)row_bytes);
  const uint32_t nvec = static_cast<uint32_t>(nvec64);
  // slot mode (see the kernel): rows of up to 4 KB whose vector count is no power of two but fills at
  // least 3/4 of the next one.  Measured with 400-byte rows: peer rows 514 -> 578 GB/s, host rows
  // 40 -> 45 GB/s, local rows unchanged.  DGS_GATHER_SLOTS=0 switches it off.
  uint32_t slot_shift = 0;
  {
    uint32_t sl = 0;
    while ((1u << sl) < nvec) ++sl;
    static const char* env = std::getenv("DGS_GATHER_SLOTS");
    const bool eligible = nvec > 2 && (1u << sl) != nvec && (1u << sl) <= 256 && 4 * nvec >= 3 * (1u << sl);
    const bool wanted = !(env != nullptr && env[0] == '0');
    if (eligible && wanted) slot_shift = sl;
  }
  uint32_t rows_per_tile =
      (GATHER_BLOCK * (REALIGN ? GATHER_UNROLL / 2 : GATHER_UNROLL)) / (slot_shift ? (1u << slot_shift) : nvec);
  if (rows_per_tile < 1) rows_per_tile = 1;
  if (rows_per_tile > GATHER_MAX_ROWS) rows_per_tile = GATHER_MAX_ROWS;
  // rows > 1 implies rows*nvec <= 2048 and nvec <= 1024, so q*nvec < 2^21 in the kernel
  const uint32_t magic =
      nvec == 1 ? 0u : static_cast<uint32_t>(((1ull << 32) + nvec - 1) / nvec);
  const int64_t tiles = (n + rows_per_tile - 1) / rows_per_tile;
  DGS_REQUIRE(tiles <= 0x7fffffffLL, DGS_ERR_UNSUPPORTED, "gather: too many rows (%lld)", (long long)n);
  DGS_CUDA_TRY(launch_chained(SITE_GATHER, gather_rows_kernel<Src, VEC, REALIGN>, static_cast<unsigned>(tiles), GATHER_BLOCK, stream, rows,
                              n, nc.dev, D, sh, nvec, rows_per_tile, magic, slot_shift, static_cast<char*>(out), status));
  return DGS_OK;
}


// ---- rows moved by the copy engine ------------------------------------------------
// The kernel above keeps its bytes in flight in registers (eight 16-byte loads per thread), which at four
// CTAs per SM is the whole register file: nothing else can run beside it.  This variant moves whole rows
// with bulk asynchronous copies instead -- one cp.async.bulk per row from wherever the row lives (local HBM,
// a peer's HBM over NVLink, pinned host memory) into shared memory, completion counted by an mbarrier, then
// ONE bulk store per group of rows, because a group's output rows are contiguous.  The bytes in flight sit in
// shared memory, a warp needs a handful of registers, and one small persistent CTA per SM is enough -- so the
// short latency-bound kernels of other mini-batches' sampling sequences run on the same SMs at the same time.
//
// Every warp is its own pipeline (no CTA-wide barrier): STAGES buffers of `group` rows each; lane l owns row
// l of the group.  Per group: resolve the row (as above), lane 0 announces the bytes to expect, every lane
// issues its row's copy; rows that cannot be copied whole (they straddle two storage regions, or the id is
// out of range) are written into the buffer by their lane with ordinary stores.  When the group has landed,
// lane 0 issues the store, and the buffer is loaded again only after that store has read it
// (cp.async.bulk.wait_group.read).  Needs rows that start on 16-byte boundaries and are a multiple of 16 bytes.
// Waits are bounded: a copy that never completes sets DGS_ERR_CUDA in the status word and the warp leaves
// after its outstanding stores.
constexpr int BULK_WARPS = 4;      // warps per CTA (the launch may choose fewer or more, up to BULK_MAX_WARPS)
constexpr int BULK_MAX_WARPS = 8;
constexpr int BULK_STAGES = 3;
constexpr uint32_t BULK_WAIT_LIMIT = 1u << 24;  // polls of ~20 ns each: a fraction of a second

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t polls = 0; polls < BULK_WAIT_LIMIT; ++polls)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// L2 policy "evict first" for data that streams through once: gathered rows and the output they are written
// to should not push the relabel tables and plan arrays of the sampling kernels (which run at the same time,
// for other mini-batches) out of the L2
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
// global -> shared, `bytes` a multiple of 16, both addresses 16-byte aligned; no multicast
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar,
                                          uint64_t policy, bool hinted) {
  if (hinted)
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            dst_smem),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
  else
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes, uint64_t policy, bool hinted) {
  if (hinted)
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(dst), "r"(src_smem),
                 "r"(bytes), "l"(policy)
                 : "memory");
  else
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
                 : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <typename Src>
__global__ void __launch_bounds__(BULK_MAX_WARPS * 32)
gather_rows_bulk_kernel(const __grid_constant__ Src rows, const int64_t n_bound, const int64_t* __restrict__ n_dev,
                        const int64_t D, const int sh, const uint32_t row_bytes, const uint32_t group,
                        const uint32_t stage_bytes, const bool l2_hint, char* __restrict__ out,
                        int32_t* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  const uint64_t policy = l2_evict_first_policy();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int n_warps = blockDim.x >> 5;
  unsigned char* my_stages = bulk_smem + static_cast<size_t>(warp) * BULK_STAGES * stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(bulk_smem + static_cast<size_t>(n_warps) * BULK_STAGES * stage_bytes) +
                   warp * BULK_STAGES;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < BULK_STAGES; ++s) mbar_init(smem_addr(bars + s), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  pdl_enter();

  int64_t n = n_bound;
  if (n_dev != nullptr) {
    const int64_t live = *n_dev;
    n = live < n_bound ? (live < 0 ? 0 : live) : n_bound;
  }
  const int64_t n_groups = (n + group - 1) / group;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * n_warps;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * n_warps + warp;

  // the row id lane `lane` will need for group g (read one iteration before the group is issued, so that
  // the warp never waits for it)
  auto fetch_id = [&](int64_t g) -> int64_t {
    const int64_t i = g * group + lane;
    return (g < n_groups && lane < static_cast<int>(group) && i < n) ? rows.row_id(i) : 0;
  };
  // loads of group g into stage st; row = what fetch_id(g) returned
  auto issue = [&](int64_t g, int st, int64_t row) {
    const int64_t i = g * group + lane;
    const bool valid = lane < static_cast<int>(group) && i < n;
    const char* src = valid ? rows.template locate_row<16, false>(row, status) : nullptr;
    const bool whole = valid && reinterpret_cast<uintptr_t>(src) > 1;
    const uint32_t bar = smem_addr(bars + st);
    unsigned char* slot = my_stages + static_cast<size_t>(st) * stage_bytes + static_cast<size_t>(lane) * row_bytes;
    const uint32_t expect = static_cast<uint32_t>(__popc(__ballot_sync(FULL_MASK, whole))) * row_bytes;
    if (lane == 0) mbar_expect_tx(bar, expect);  // also the one arrival the barrier waits for
    __syncwarp();
    if (whole) {
      bulk_load(smem_addr(slot), src, row_bytes, bar, policy, l2_hint);
    } else if (valid) {
      // rare: zero row (bad id) or a row that straddles two storage regions, element by element
      const int esz = 1 << sh;
      if (src == DGS_ROW_ZERO) {
        for (uint32_t b = 0; b < row_bytes; b += 16) *reinterpret_cast<uint4*>(slot + b) = make_uint4(0u, 0u, 0u, 0u);
      } else {
        for (int64_t j = 0; j < D; ++j) {
          const char* p = rows.element(i, j);
          unsigned char* q = slot + (j << sh);
          switch (esz) {
            case 8: *reinterpret_cast<uint64_t*>(q) = *reinterpret_cast<const uint64_t*>(p); break;
            case 4: *reinterpret_cast<uint32_t*>(q) = *reinterpret_cast<const uint32_t*>(p); break;
            case 2: *reinterpret_cast<uint16_t*>(q) = *reinterpret_cast<const uint16_t*>(p); break;
            default: *q = static_cast<unsigned char>(*p); break;
          }
        }
      }
      fence_async_smem();  // these ordinary stores must be visible to the bulk store that reads the buffer
    }
  };

  // prologue: STAGES - 1 groups ahead
  int64_t g_issue = first;
#pragma unroll
  for (int s = 0; s < BULK_STAGES - 1; ++s) {
    if (g_issue < n_groups) issue(g_issue, s, fetch_id(g_issue));
    g_issue += stride;
  }
  int64_t next_row = fetch_id(g_issue);  // for the group the first iteration will issue
  uint32_t phase_bits = 0;  // parity of each stage's barrier
  int st = 0, st_issue = BULK_STAGES - 1;
  bool alive = true;
  for (int64_t g = first; g < n_groups && alive; g += stride) {
    const uint32_t bar = smem_addr(bars + st);
    if (!mbar_wait_bounded(bar, (phase_bits >> st) & 1u)) {
      raise_status(status, DGS_ERR_CUDA);
      alive = false;
    }
    alive = __all_sync(FULL_MASK, alive);
    if (!alive) break;
    __syncwarp();  // rows that lanes wrote into the buffer themselves are visible to lane 0's store
    phase_bits ^= 1u << st;
    if (lane == 0) {
      const int64_t row0 = g * group;
      const int64_t rows_here = n - row0 < static_cast<int64_t>(group) ? n - row0 : static_cast<int64_t>(group);
      bulk_store(out + row0 * row_bytes, smem_addr(my_stages + static_cast<size_t>(st) * stage_bytes),
                 static_cast<uint32_t>(rows_here) * row_bytes, policy, l2_hint);
      // the buffer that is loaded next was stored from one iteration ago: that store must have read it
      bulk_wait_read<1>();
    }
    __syncwarp();
    const int64_t row_now = next_row;
    next_row = fetch_id(g_issue + stride);  // in flight while this iteration's copies are issued and awaited
    if (g_issue < n_groups) issue(g_issue, st_issue, row_now);
    g_issue += stride;
    st = st + 1 == BULK_STAGES ? 0 : st + 1;
    st_issue = st_issue + 1 == BULK_STAGES ? 0 : st_issue + 1;
  }
  if (!alive) {
    // give the copies still in flight a bounded chance to land before the buffers go away
    for (int s = 0; s < BULK_STAGES; ++s) mbar_wait_bounded(smem_addr(bars + s), (phase_bits >> s) & 1u);
  }
  if (lane == 0) bulk_wait_all();  // shared memory must outlive the stores that read it
}

// rows a warp moves per group and the bytes of one buffer, for rows of row_bytes
inline void bulk_geometry(int64_t row_bytes, uint32_t* group, uint32_t* stage_bytes) {
  // 8 KB per buffer: measured on 400-byte rows, 4 warps x 3 buffers x 8 KB (96 KB in flight per SM) reaches the
  // DRAM rate of the register form; half of that (4 KB buffers) gives 0.61 instead of 0.74 of the HBM peak,
  // and more warps or larger buffers gain nothing alone and cost the sampling kernels beside it their room
  uint32_t g = static_cast<uint32_t>(8192 / row_bytes);
  if (g > 32) g = 32;
  if (g < 1) g = 1;
  *group = g;
  *stage_bytes = (g * static_cast<uint32_t>(row_bytes) + 127u) / 128u * 128u;
}

// DGS_GATHER_BULK: 0 = never, 1 = whenever the rows qualify, unset = the default of the call site
inline int bulk_env() {
  static const int v = [] {
    const char* e = std::getenv("DGS_GATHER_BULK");
    return e == nullptr ? -1 : (e[0] == '1' ? 1 : 0);
  }();
  return v;
}

template <typename Src>
int launch_gather_bulk(const Src& rows, Count nc, int64_t D, int sh, void* out, int32_t* status, cudaStream_t stream) {
  const int64_t row_bytes = D << sh;
  uint32_t group, stage_bytes;
  bulk_geometry(row_bytes, &group, &stage_bytes);
  constexpr int warps = BULK_WARPS;
  const size_t smem = static_cast<size_t>(warps) * BULK_STAGES * stage_bytes + warps * BULK_STAGES * sizeof(uint64_t);
  DGS_REQUIRE(smem <= 200 * 1024, DGS_ERR_UNSUPPORTED, "gather: %zu bytes of shared memory per CTA", smem);
  // per device and safe to reach from several host threads: the SM count, and whether this instantiation has
  // been allowed its dynamic shared memory there (the attribute belongs to the device's copy of the kernel)
  constexpr int kMaxDevices = 64;
  static std::atomic<int> sm_count[kMaxDevices] = {};
  static std::atomic<bool> smem_opted_in[kMaxDevices] = {};
  int dev = 0;
  DGS_CUDA_TRY(cudaGetDevice(&dev));
  DGS_REQUIRE(dev >= 0 && dev < kMaxDevices, DGS_ERR_UNSUPPORTED, "gather: device ordinal %d", dev);
  int sms = sm_count[dev].load(std::memory_order_relaxed);
  if (sms == 0) {
    DGS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    sm_count[dev].store(sms, std::memory_order_relaxed);
  }
  // one persistent CTA per SM (two per SM: 0.70 instead of 0.68 alone, but the pipelined step got slower)
  const int64_t groups = (nc.bound + group - 1) / group;
  int64_t grid = (groups + warps - 1) / warps;
  if (grid > static_cast<int64_t>(sms)) grid = static_cast<int64_t>(sms);
  auto kernel = gather_rows_bulk_kernel<Src>;
  if (!smem_opted_in[dev].load(std::memory_order_acquire)) {  // the buffers never exceed 12 x 8 KB + the barriers
    DGS_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    smem_opted_in[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(warps * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launches_enabled(SITE_GATHER) ? 1 : 0;
  constexpr bool l2_hint = true;  // evict-first: 0.80 instead of 0.76 of the HBM peak at 1 M rows, same in the pipeline
  DGS_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, rows, nc.bound, nc.dev, D, sh, static_cast<uint32_t>(row_bytes), group,
                                  stage_bytes, l2_hint, static_cast<char*>(out), status));
  return DGS_OK;
}

inline bool bulk_rows_qualify(int vec, bool realign, int64_t row_bytes) {
  return vec == 16 && !realign && (row_bytes % 16) == 0 && row_bytes >= 256 && row_bytes <= 8192;
}

// realign: some storage region starts rows off the vector boundary (see vector_copy_ok)
template <typename Src, int VEC>
int launch_gather(const Src& rows, bool realign, Count n, int64_t D, int sh, void* out, int32_t* status,
                  cudaStream_t stream) {
  if constexpr (VEC >= 8) {
    if (realign) return launch_gather_r<Src, VEC, true>(rows, n, D, sh, out, status, stream);
  }
  return launch_gather_r<Src, VEC, false>(rows, n, D, sh, out, status, stream);
}

template <typename Src>
int dispatch_vec(int vec, bool realign, const Src& rows, Count n, int64_t D, int sh, void* out,
                 int32_t* status, cudaStream_t stream) {
  switch (vec) {
    case 16: return launch_gather<Src, 16>(rows, realign, n, D, sh, out, status, stream);
    case 8: return launch_gather<Src, 8>(rows, realign, n, D, sh, out, status, stream);
    case 4: return launch_gather<Src, 4>(rows, false, n, D, sh, out, status, stream);
    case 2: return launch_gather<Src, 2>(rows, false, n, D, sh, out, status, stream);
    default: return launch_gather<Src, 1>(rows, false, n, D, sh, out, status, stream);
  }
}

// prefer_bulk: what the call site wants when DGS_GATHER_BULK does not say
template <typename IdxT>
int run_gather(int vec, bool realign, const dgs_chunk_desc& d, const void* idx, Count n, int64_t D, int sh,
               void* out, int32_t* status, bool prefer_bulk, cudaStream_t stream) {
  ChunkRows<IdxT> rows{d, static_cast<const IdxT*>(idx), D, d.total / D, sh};
  const int env = bulk_env();
  if ((env == 1 || (env < 0 && prefer_bulk)) && bulk_rows_qualify(vec, realign, D << sh))
    return launch_gather_bulk(rows, n, D, sh, out, status, stream);
  return dispatch_vec(vec, realign, rows, n, D, sh, out, status, stream);
}

// ---- cache table build -------------------------------------------------------
// Replaces CreateHashMapTensorCUDA's insert pass (reference src/cuda/pagraph.cu:94-124).
template <typename IdT>
__global__ void __launch_bounds__(256)
cache_build_kernel(const IdT* __restrict__ keys, const IdT* __restrict__ values, const int64_t n,
                   IdT* key_buf, IdT* value_buf, const uint64_t mask, int32_t* __restrict__ status) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n) return;
  const IdT key = keys[i];
  if (key < 0) {
    raise_status(status, DGS_ERR_RANGE);
    return;
  }
  uint64_t h = cache_hash(static_cast<long long>(key)) & mask;
  for (uint64_t probes = 0; probes <= mask; ++probes) {
    IdT cur = *reinterpret_cast<volatile IdT*>(&key_buf[h]);
    if (cur == static_cast<IdT>(-1)) {
      if (sizeof(IdT) == 8)
        cur = static_cast<IdT>(atomicCAS(reinterpret_cast<unsigned long long*>(&key_buf[h]),
                                         ~0ull, static_cast<unsigned long long>(key)));
      else
        cur = static_cast<IdT>(atomicCAS(reinterpret_cast<unsigned int*>(&key_buf[h]), ~0u,
                                         static_cast<unsigned int>(key)));
    }
    if (cur == static_cast<IdT>(-1) || cur == key) {
      value_buf[h] = values[i];  // duplicates: last writer wins, as in the reference (:27)
      return;
    }
    h = (h + 1) & mask;
  }
  raise_status(status, DGS_ERR_TABLE_FULL);
}

template <typename IdxT>
int run_cache_fetch(int vec, bool realign, const dgs_chunk_desc& gpu, const void* cpu_data, int64_t cpu_rows,
                    const void* nid,
                    const void* keys, const void* values, int64_t slots, int64_t n, int64_t D,
                    int sh, void* out, int32_t* status, cudaStream_t stream) {
  CachedRows<IdxT> rows{gpu,
                        static_cast<const char*>(cpu_data),
                        static_cast<const IdxT*>(nid),
                        static_cast<const IdxT*>(keys),
                        static_cast<const IdxT*>(values),
                        static_cast<uint64_t>(slots - 1),
                        D,
                        gpu.total / D,
                        cpu_rows,
                        sh};
  return dispatch_vec(vec, realign, rows, exact_count(n), D, sh, out, status, stream);
}

// largest power of two <= 16 dividing x (x == 0 counts as "any")
inline int pow2_div(uint64_t x) {
  int v = 16;
  while (v > 1 && (x % static_cast<uint64_t>(v)) != 0) v >>= 1;
  return v;
}

}  // namespace

int validate_desc(const dgs_chunk_desc* t, const char* who) {
  DGS_REQUIRE(t != nullptr, DGS_ERR_INVALID, "%s: null descriptor", who);
  DGS_REQUIRE(esz_log2(t->esz) >= 0, DGS_ERR_UNSUPPORTED, "%s: element size %d", who, t->esz);
  DGS_REQUIRE(t->num_parts >= 1 && t->num_parts <= DGS_MAX_PARTS, DGS_ERR_INVALID,
              "%s: num_parts %d outside 1..%d", who, t->num_parts, DGS_MAX_PARTS);
  DGS_REQUIRE(t->total >= 0 && t->threshold >= 0 && t->threshold <= t->total && t->each >= 0,
              DGS_ERR_INVALID, "%s: inconsistent sizes", who);
  DGS_REQUIRE(t->threshold <= t->each * t->num_parts, DGS_ERR_INVALID,
              "%s: threshold exceeds each*num_parts", who);
  DGS_REQUIRE(t->threshold == t->total || t->host != nullptr, DGS_ERR_INVALID,
              "%s: host tail missing", who);
  if (t->threshold > 0)
    for (int p = 0; p * t->each < t->threshold; ++p)
      DGS_REQUIRE(t->dev[p] != nullptr, DGS_ERR_INVALID, "%s: chunk %d has no pointer", who, p);
  return DGS_OK;
}

// Vector width of the copy.  The row size and the output decide it; where the storage regions start
// (chunk bases, `each`, `threshold`) only lowers it when rows that start off the vector boundary cannot be
// realigned in the kernel (elements below 4 bytes, offsets that are no whole words).  *realign is set when
// the kernel has to be the realigning instance.
int gather_vec_bytes(const dgs_chunk_desc& d, int64_t D, const void* out, bool* realign) {
  const int sh = esz_log2(d.esz);
  uint64_t g = static_cast<uint64_t>(D) << sh;  // row bytes
  const int v_row = min(pow2_div(g), pow2_div(reinterpret_cast<uintptr_t>(out)));
  int v_regions = 16;
  if (d.threshold > 0) {
    for (int p = 0; p * d.each < d.threshold; ++p)
      v_regions = min(v_regions, pow2_div(reinterpret_cast<uintptr_t>(d.dev[p])));
    if (d.threshold > d.each) v_regions = min(v_regions, pow2_div(static_cast<uint64_t>(d.each) << sh));
  }
  if (d.threshold < d.total) {
    v_regions = min(v_regions, pow2_div(reinterpret_cast<uintptr_t>(d.host)));
    v_regions = min(v_regions, pow2_div(static_cast<uint64_t>(d.threshold) << sh));
  }
  *realign = false;
  if (v_regions >= v_row) return v_row;
  // Measured on B200 (512-byte rows, 90 % local / 10 % host): regions on 8-byte boundaries -- 8-byte vectors
  // throughout give 0.95 of the HBM rate for local and 0.77 of the link rate for host rows, the realigning
  // instance 0.60 / 0.77 (it halves the loads in flight and shuffles every vector); regions on 4-byte
  // boundaries -- 4-byte vectors give 0.60 / 0.62, the realigning instance 0.60 / 0.76.  So it is used for
  // the second case only.  DGS_GATHER_REALIGN=0 switches it off.
  static const char* env = std::getenv("DGS_GATHER_REALIGN");
  if (d.esz >= 4 && v_row >= 8 && v_regions == 4 && !(env != nullptr && env[0] == '0')) {
    *realign = true;
    return v_row;
  }
  return v_regions;
}

}  // namespace dgs

namespace dgs {
namespace {
int gather_entry(const char* who, const dgs_chunk_desc* t, const void* idx, int32_t ids64, Count n, int64_t D,
                 void* out, int32_t* status, bool prefer_bulk, dgs_stream_t stream) {
  int rc = validate_desc(t, who);
  if (rc != DGS_OK) return rc;
  DGS_REQUIRE(n.bound >= 0 && D >= 1, DGS_ERR_INVALID, "%s: n=%lld D=%lld", who, (long long)n.bound, (long long)D);
  if (n.bound == 0) return DGS_OK;
  DGS_REQUIRE(idx != nullptr && out != nullptr, DGS_ERR_INVALID, "%s: null buffer", who);
  const int sh = esz_log2(t->esz);
  bool realign = false;
  const int vec = gather_vec_bytes(*t, D, out, &realign);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ids64 ? run_gather<int64_t>(vec, realign, *t, idx, n, D, sh, out, status, prefer_bulk, s)
               : run_gather<int32_t>(vec, realign, *t, idx, n, D, sh, out, status, prefer_bulk, s);
}
}  // namespace
}  // namespace dgs

extern "C" int dgs_gather_rows(const dgs_chunk_desc* t, int32_t location_class, const void* idx,
                               int32_t ids64, int64_t n, int64_t D, void* out, int32_t* status,
                               dgs_stream_t stream) {
  (void)location_class;  // hint only: the owner is resolved per row for every class
  return dgs::gather_entry("dgs_gather_rows", t, idx, ids64, dgs::exact_count(n), D, out, status, false, stream);
}

extern "C" int dgs_gather_rows_counted(const dgs_chunk_desc* t, const void* idx, int32_t ids64, int64_t n_bound,
                                       const int64_t* n_dev, int64_t D, void* out, int32_t* status,
                                       dgs_stream_t stream) {
  using namespace dgs;
  DGS_REQUIRE(n_dev != nullptr, DGS_ERR_INVALID, "dgs_gather_rows_counted: null row count");
  // queued behind a sampling sequence while other mini-batches are in flight: the form that shares the SMs
  return gather_entry("dgs_gather_rows_counted", t, idx, ids64, Count{n_bound, n_dev, nullptr}, D, out, status, true, stream);
}

extern "C" int64_t dgs_cache_table_slots(int64_t n_keys) {
  // same growth rule as the reference (2 * next power of two above n, pagraph.cu:89-101)
  int64_t p = 1;
  while (p <= n_keys) p <<= 1;
  return 2 * p;
}

extern "C" int dgs_cache_build(const void* keys, const void* values, int32_t ids64, int64_t n_keys,
                               void* key_buf, void* value_buf, int64_t slots, int32_t* status,
                               dgs_stream_t stream) {
  using namespace dgs;
  DGS_REQUIRE(n_keys >= 0 && slots >= 2 && (slots & (slots - 1)) == 0 && slots > n_keys, DGS_ERR_INVALID,
              "dgs_cache_build: slots=%lld must be a power of two above n_keys=%lld", (long long)slots,
              (long long)n_keys);
  DGS_REQUIRE(key_buf != nullptr && value_buf != nullptr, DGS_ERR_INVALID, "dgs_cache_build: null table");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t esz = ids64 ? 8 : 4;
  // empty key = -1; untouched values read as the id type's maximum like the reference's fill (:104-107)
  DGS_CUDA_TRY(cudaMemsetAsync(key_buf, 0xFF, static_cast<size_t>(slots) * esz, s));
  DGS_CUDA_TRY(cudaMemsetAsync(value_buf, 0x7F, static_cast<size_t>(slots) * esz, s));
  if (n_keys == 0) return DGS_OK;
  DGS_REQUIRE(keys != nullptr && values != nullptr, DGS_ERR_INVALID, "dgs_cache_build: null input");
  const unsigned grid = static_cast<unsigned>((n_keys + 255) / 256);
  if (ids64)
    cache_build_kernel<int64_t><<<grid, 256, 0, s>>>(static_cast<const int64_t*>(keys),
                                                     static_cast<const int64_t*>(values), n_keys,
                                                     static_cast<int64_t*>(key_buf),
                                                     static_cast<int64_t*>(value_buf),
                                                     static_cast<uint64_t>(slots - 1), status);
  else
    cache_build_kernel<int32_t><<<grid, 256, 0, s>>>(static_cast<const int32_t*>(keys),
                                                     static_cast<const int32_t*>(values), n_keys,
                                                     static_cast<int32_t*>(key_buf),
                                                     static_cast<int32_t*>(value_buf),
                                                     static_cast<uint64_t>(slots - 1), status);
  DGS_LAUNCH_CHECK();
  return DGS_OK;
}

extern "C" int dgs_cache_fetch(const void* cpu_data, int64_t cpu_rows,
                               const dgs_chunk_desc* gpu_data, const void* nid,
                               int32_t ids64, int64_t n, int64_t D, const void* key_buf,
                               const void* value_buf, int64_t slots, void* out, int32_t* status,
                               dgs_stream_t stream) {
  using namespace dgs;
  int rc = validate_desc(gpu_data, "dgs_cache_fetch");
  if (rc != DGS_OK) return rc;
  DGS_REQUIRE(n >= 0 && D >= 1 && slots >= 2 && (slots & (slots - 1)) == 0, DGS_ERR_INVALID,
              "dgs_cache_fetch: bad arguments");
  if (n == 0) return DGS_OK;
  DGS_REQUIRE(cpu_data != nullptr && nid != nullptr && key_buf != nullptr && value_buf != nullptr &&
                  out != nullptr,
              DGS_ERR_INVALID, "dgs_cache_fetch: null buffer");
  const int sh = esz_log2(gpu_data->esz);
  bool realign = false;
  int vec = gather_vec_bytes(*gpu_data, D, out, &realign);
  vec = min(vec, pow2_div(reinterpret_cast<uintptr_t>(cpu_data)));
  if (vec < 8) realign = false;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ids64 ? run_cache_fetch<int64_t>(vec, realign, *gpu_data, cpu_data, cpu_rows, nid, key_buf, value_buf, slots, n, D,
                                          sh, out, status, s)
               : run_cache_fetch<int32_t>(vec, realign, *gpu_data, cpu_data, cpu_rows, nid, key_buf, value_buf, slots, n, D,
                                          sh, out, status, s);
}
