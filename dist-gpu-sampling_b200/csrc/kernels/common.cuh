// Shared device/host helpers for the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/dgs_b200.h"

namespace dgs {

// ---- host-side error plumbing (defined in host/error.cc) -------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define DGS_CUDA_TRY(call)                                             \
  do {                                                                 \
    cudaError_t e__ = (call);                                          \
    if (e__ != cudaSuccess) return ::dgs::cuda_fail(e__, #call, __FILE__, __LINE__); \
  } while (0)

#define DGS_LAUNCH_CHECK()                                             \
  do {                                                                 \
    cudaError_t e__ = cudaGetLastError();                              \
    if (e__ != cudaSuccess) return ::dgs::cuda_fail(e__, "kernel launch", __FILE__, __LINE__); \
  } while (0)

#define DGS_REQUIRE(cond, code, ...)      \
  do {                                    \
    if (!(cond)) {                        \
      ::dgs::set_error(__VA_ARGS__);      \
      return (code);                      \
    }                                     \
  } while (0)

// descriptor sanity checks shared by all launchers (defined in gather.cu)
int validate_desc(const dgs_chunk_desc* t, const char* who);

static inline int esz_log2(int32_t esz) {
  switch (esz) {
    case 1: return 0;
    case 2: return 1;
    case 4: return 2;
    case 8: return 3;
    default: return -1;
  }
}

// A number of items that the host knows exactly (dev == nullptr: it is `bound`)
// or only as an upper bound, the exact value being the sum of one or two device
// words written by an earlier kernel on the same stream.  Launch grids are sized
// by `bound`; kernels work on count_of().  This is what lets a whole multi-hop
// sample -> relabel sequence be queued without the host reading a size back.
struct Count {
  int64_t bound;
  const int64_t* dev;
  const int64_t* dev2;
};
static inline Count exact_count(int64_t n) { return Count{n, nullptr, nullptr}; }

// The Philox key of one sampling launch: a value the host computed, or (dev != nullptr) a device word an
// earlier kernel of the same stream wrote -- what a recorded launch sequence needs, whose parameters are
// fixed while its random stream changes from replay to replay.
struct RngKey {
  uint64_t value;
  const uint64_t* dev;
};
static inline RngKey host_key(uint64_t v) { return RngKey{v, nullptr}; }

#ifdef __CUDACC__

constexpr unsigned FULL_MASK = 0xffffffffu;

// ---- chained launches ----------------------------------------------------------
// Kernels that follow one another on a stream are launched with programmatic
// stream serialization: the next kernel's CTAs may be placed on the SMs while the
// previous kernel drains, which takes the launch latency out of a chain of short
// dependent kernels.  Every such kernel starts with pdl_enter(): it waits until
// the previous kernel has completed and its writes are visible (so nothing about
// the data flow changes) and then lets its own successor be placed.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// which launch this is; DGS_NO_PDL=1 turns the attribute off everywhere, DGS_PDL_OFF_MASK=<hex> per site
enum LaunchSite { SITE_INIT = 0, SITE_PLAN, SITE_SAMPLE, SITE_INSERT, SITE_COUNT, SITE_NUMBER, SITE_LOOKUP,
                  SITE_GATHER, SITE_CLEAR };
bool chained_launches_enabled(int site);  // host/error.cc

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(int site, void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t s,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launches_enabled(site) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ int64_t count_of(const Count& c) {
  if (c.dev == nullptr) return c.bound;
  int64_t v = *c.dev;
  if (c.dev2 != nullptr) v += *c.dev2;
  return v < c.bound ? (v < 0 ? 0 : v) : c.bound;
}

__device__ __forceinline__ uint64_t key_of(const RngKey& k) { return k.dev == nullptr ? k.value : *k.dev; }

// Sticky status word: first error wins, later ones are dropped.
__device__ __forceinline__ void raise_status(int32_t* status, int32_t code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// ---- ChunkTensor element resolution ----------------------------------------
// Pointer to flat element e (0 <= e < d.total) and, in *run, how many elements
// starting at e are contiguous in the same storage region.
// Same mapping as chunk_tensor_wrapper<T>::At (reference src/chunk_tensor.h:33-42)
// but on a by-value descriptor: no metadata loads, no 64-bit divide (the owner
// is found with at most num_parts-1 compares).
__device__ __forceinline__ const char* resolve(const dgs_chunk_desc& d, int sh, int64_t e,
                                               int64_t* run) {
  if (e >= d.threshold) {
    *run = d.total - e;
    return static_cast<const char*>(d.host) + ((e - d.threshold) << sh);
  }
  int p = 0;
  int64_t base = 0;
  int64_t b = d.each;
#pragma unroll
  for (int q = 1; q < DGS_MAX_PARTS; ++q) {
    if (q >= d.num_parts) break;  // uniform: a plain tensor (one part) skips the chain
    if (e >= b) {
      p = q;
      base = b;
    }
    b += d.each;
  }
  int64_t end = base + d.each;
  if (end > d.threshold) end = d.threshold;
  *run = end - e;
  return static_cast<const char*>(d.dev[p]) + ((e - base) << sh);
}

template <typename T>
__device__ __forceinline__ T load_at(const dgs_chunk_desc& d, int sh, int64_t e) {
  int64_t run;
  return *reinterpret_cast<const T*>(resolve(d, sh, e, &run));
}

// Read-only, L1-bypassing loads for streamed rows (local HBM, peer HBM over
// NVLink, or pinned host memory: all plain global-space addresses under UVA).
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_stream(const uint2* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_stream(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint16_t ld_stream(const uint16_t* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint8_t ld_stream(const uint8_t* p) { return *p; }

// ---- block-wide exclusive scan ----------------------------------------------
// BLOCK threads, one value each.  `smem` needs BLOCK/32 + 1 entries of T.
// Returns the exclusive prefix of the caller's value; *total = block sum.
template <typename T, int BLOCK>
__device__ __forceinline__ T block_exclusive_scan(T v, T* smem, T* total) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  T inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    T t = __shfl_up_sync(FULL_MASK, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) smem[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    constexpr int NW = BLOCK / 32;
    T w = (lane < NW) ? smem[lane] : T(0);
    T winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      T t = __shfl_up_sync(FULL_MASK, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < NW) smem[lane] = winc - w;  // exclusive warp offsets
    if (lane == NW - 1) smem[NW] = winc;   // block total
  }
  __syncthreads();
  T res = smem[warp] + inc - v;
  *total = smem[BLOCK / 32];
  __syncthreads();  // smem may be reused by the caller
  return res;
}

// ---- segments (logical concatenation of device arrays) ----------------------
template <typename IdT>
__device__ __forceinline__ IdT seg_load(const dgs_segments& s, int64_t i) {
  int q = 0;
  int64_t base = 0;
#pragma unroll
  for (int j = 0; j < DGS_MAX_SEGMENTS - 1; ++j) {
    if (j + 1 < s.count && i >= base + s.len[j]) {
      base += s.len[j];
      q = j + 1;
    } else {
      break;
    }
  }
  return static_cast<const IdT*>(s.ptr[q])[i - base];
}

#endif  // __CUDACC__
}  // namespace dgs
