// Counter-based Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy
// as 1, 2, 3", SC'11), written from the published algorithm.  Replaces the
// cuRAND Philox state the reference initialises per thread with a constant
// seed (src/cuda/rowwise_sampling.cu:57-58,152): here every draw is a pure
// function of (key, counter), so no state is carried and no curand_init runs.
#pragma once
#include <stdint.h>

namespace dgs {

struct Philox4 {
  uint32_t x, y, z, w;
};

#ifdef __CUDACC__
#define DGS_HD __host__ __device__ __forceinline__
#else
#define DGS_HD inline
#endif

DGS_HD void philox_mulhilo(uint32_t a, uint32_t b, uint32_t* hi, uint32_t* lo) {
  uint64_t p = static_cast<uint64_t>(a) * b;
  *hi = static_cast<uint32_t>(p >> 32);
  *lo = static_cast<uint32_t>(p);
}

DGS_HD Philox4 philox4x32_10(uint64_t key, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(M0, c0, &hi0, &lo0);
    philox_mulhilo(M1, c2, &hi1, &lo1);
    uint32_t n0 = hi1 ^ c1 ^ k0;
    uint32_t n1 = lo1;
    uint32_t n2 = hi0 ^ c3 ^ k1;
    uint32_t n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0;
    k1 += W1;
  }
  Philox4 o;
  o.x = c0; o.y = c1; o.z = c2; o.w = c3;
  return o;
}

// splitmix64 finaliser; used on the host to fold (seed, offset) into one key.
DGS_HD uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// (seed, offset) of a random stream folded into the Philox key of one sampling launch; the same on the
// host (launch parameter) and on the device (a recorded sequence reads seed and offset when it runs).
DGS_HD uint64_t fold_rng_key(uint64_t rng_seed, uint64_t rng_offset) {
  return mix64(rng_seed) ^ mix64(rng_offset ^ 0xA5A5A5A55A5A5A5Aull);
}

// Unbiased integer in [0, n), n >= 1, from one Philox block (Lemire's
// multiply-shift with rejection; the reference's `curand() % n` is biased).
// The four 32-bit words are four successive attempts; a fifth rejection has
// probability < (n/2^32)^4 and is accepted as is.
DGS_HD uint64_t bounded(const Philox4& r, uint64_t n) {
  if (n <= 0xFFFFFFFFull) {
    const uint32_t n32 = static_cast<uint32_t>(n);
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
    uint64_t m = 0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      m = static_cast<uint64_t>(w[t]) * n32;
      // the rejection threshold 2^32 mod n costs a division, so it is only
      // computed in the rare case (probability n / 2^32) where it can matter
      if (static_cast<uint32_t>(m) >= n32 || static_cast<uint32_t>(m) >= (0u - n32) % n32) break;
    }
    return m >> 32;
  }
  // rows longer than 2^32 edges: 64-bit variant, two attempts
  const uint64_t thresh = (0ull - n) % n;
  uint64_t r0 = (static_cast<uint64_t>(r.x) << 32) | r.y;
  uint64_t r1 = (static_cast<uint64_t>(r.z) << 32) | r.w;
#ifdef __CUDA_ARCH__
  uint64_t hi = __umul64hi(r0, n), lo = r0 * n;
  if (lo < thresh) { hi = __umul64hi(r1, n); }
  return hi;
#else
  unsigned __int128 p = static_cast<unsigned __int128>(r0) * n;
  if (static_cast<uint64_t>(p) < thresh) p = static_cast<unsigned __int128>(r1) * n;
  return static_cast<uint64_t>(p >> 64);
#endif
}

// One attempt of the same method on a single 32-bit word (n < 2^32): returns
// false when the word falls into the rejection zone and must be replaced.
DGS_HD bool bounded_try(uint32_t word, uint32_t n32, uint32_t* out) {
  const uint64_t m = static_cast<uint64_t>(word) * n32;
  *out = static_cast<uint32_t>(m >> 32);
  const uint32_t lo = static_cast<uint32_t>(m);
  return lo >= n32 || lo >= (0u - n32) % n32;
}

// uniform float in (0, 1] from 24 random bits (same open/closed ends as
// curand_uniform, which the reference's weighted kernels call).
DGS_HD float unit_float(uint32_t r) { return (static_cast<float>(r >> 8) + 1.0f) * (1.0f / 16777216.0f); }

}  // namespace dgs
