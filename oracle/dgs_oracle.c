/*
 * dgs_oracle.c -- CPU restatement of the Dist-GPU-sampling hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library
 * and the timed CPU baseline; nothing in the product links or calls it.
 *
 * The reference (gpzlx1/Dist-GPU-sampling) has no CPU implementation of any
 * operator -- every op rejects non-CUDA inputs (src/dgs_headers.h:4-7) -- so
 * each function below restates, in plain C, the arithmetic of the CUDA source
 * it cites.  Parity status:
 *   - placement / host-tail layout: pinned by the reference's only golden
 *     vector, the demo output in README.md:48-63 (example/demo.py:24-36).
 *   - index, split-index, local/host index, relabel (int64 and int32, absent
 *     ids), sampling of rows with deg <= fan-out, per-seed grouping with and
 *     without replacement, cache fetch: pinned by outputs of the reference's
 *     own kernels, compiled for sm_100a (oracle/build_reference.sh) and run on
 *     a B200 (tests/golden/make_reference_golden.py ->
 *     tests/golden/reference_b200.json; checked by tests/test_reference_golden.py).
 *   - rows with deg > fan-out are stochastic in the reference (and re-seeded
 *     with a constant there): compared by validity and distribution only.
 *
 * Ids are int64 throughout (int32 callers widen).  Build: see oracle/Makefile.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define MIN_(a, b) ((a) < (b) ? (a) : (b))

int dgs_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1 to their children; the timed CPU baseline asks
 * for the host's cores explicitly instead of inheriting that. */
void dgs_oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------
 * Placement: src/chunk_tensor.cc:53-73.
 *   each = cap / esz; thr = each * W; if thr > total { thr = total;
 *   each = ceil(total / W); }  host = total - thr.
 * ---------------------------------------------------------------------- */
void dgs_oracle_placement(int64_t total, int32_t esz, int64_t cap_bytes, int32_t world,
                          int64_t* each, int64_t* thr, int64_t* host) {
  int64_t e = cap_bytes / esz;
  int64_t t = e * world;
  if (t > total) {
    t = total;
    e = (total + world - 1) / world;
  }
  *each = e;
  *thr = t;
  *host = total - t;
}

/* ------------------------------------------------------------------------
 * LoadFromTensor: src/chunk_tensor.cc:173-200.  Chunk i receives flat bytes
 * [i*each, min((i+1)*each, total)); the tail after each*W goes to the host
 * buffer.  (The reference passes a negative size to cudaMemcpy when a later
 * chunk is empty; the restatement clamps at 0.)  dev[i] buffers hold `each`
 * elements and are pre-filled by the caller with 0xFF as the reference's
 * cudaMemset(-1) does (src/chunk_tensor.cc:108).
 * ---------------------------------------------------------------------- */
void dgs_oracle_load(const void* flat, int64_t total, int32_t esz, int64_t each,
                     int64_t thr, int32_t world, void** dev, void* host) {
  const char* src = (const char*)flat;
  for (int32_t i = 0; i < world; ++i) {
    int64_t lo = (int64_t)i * each;
    int64_t n = MIN_(each, total - lo);
    if (n > 0) memcpy(dev[i], src + lo * esz, (size_t)(n * esz));
  }
  if (total - thr > 0) memcpy(host, src + each * world * esz, (size_t)((total - thr) * esz));
}

/* chunk_tensor_wrapper<T>::At, src/chunk_tensor.h:33-42. */
static inline const char* at_ptr(void* const* dev, const void* host, int64_t each, int64_t thr,
                                 int32_t esz, int64_t e) {
  if (e >= thr) return (const char*)host + (e - thr) * esz;
  int64_t p = e / each;
  return (const char*)dev[p] + (e - each * p) * esz;
}

/* ------------------------------------------------------------------------
 * _IndexMemcpyKernel: src/cuda/index_with_chunk_tensor.cu:9-27.
 *   out[i*D + j] = At(index[i]*D + j)
 * ---------------------------------------------------------------------- */
void dgs_oracle_index(void* const* dev, const void* host, int64_t each, int64_t thr,
                      int32_t esz, const int64_t* idx, int64_t n, int64_t D, void* out) {
  char* o = (char*)out;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t e0 = idx[i] * D;
    for (int64_t j = 0; j < D; ++j)
      memcpy(o + (i * D + j) * esz, at_ptr(dev, host, each, thr, esz, e0 + j), (size_t)esz);
  }
}

/* Same gather on the flat logical tensor (== torch.index_select(T, 0, idx)):
 * the form used for the timed CPU baseline. */
void dgs_oracle_index_flat(const void* flat, int32_t esz, const int64_t* idx, int64_t n,
                           int64_t D, void* out) {
  const char* s = (const char*)flat;
  char* o = (char*)out;
  size_t rb = (size_t)(D * esz);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) memcpy(o + i * rb, s + idx[i] * rb, rb);
}

/* ------------------------------------------------------------------------
 * _GetSplitIndexMaskKernel + the three boolean-mask selects:
 * src/cuda/index_with_chunk_tensor.cu:55-108.  Integer divisions as written.
 * ---------------------------------------------------------------------- */
void dgs_oracle_split_index(const int64_t* idx, int64_t n, int64_t D, int64_t each,
                            int64_t thr, int64_t rank, int64_t* out_local,
                            int64_t* out_remote, int64_t* out_host, int64_t* counts) {
  int64_t nl = 0, nr = 0, nh = 0;
  for (int64_t i = 0; i < n; ++i) {
    int64_t r = idx[i];
    if (r >= thr / D) {
      out_host[nh++] = r;
    } else if (r >= rank * each / D && r < (rank + 1) * each / D) {
      out_local[nl++] = r;
    } else {
      out_remote[nr++] = r;
    }
  }
  counts[0] = nl;
  counts[1] = nr;
  counts[2] = nh;
}

/* ------------------------------------------------------------------------
 * Counter-based generator for the stochastic rows of the oracle (splitmix64
 * finaliser over (seed, row position, draw)).  The reference seeds cuRAND
 * Philox with a constant (src/cuda/rowwise_sampling.cu:57-58,152); stochastic
 * rows are compared by validity and distribution, never bit for bit, so the
 * generator itself is not part of the contract.
 * ---------------------------------------------------------------------- */
static inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
typedef struct {
  uint64_t s;
} orng;
static inline orng orng_init(uint64_t seed, uint64_t pos) {
  orng r;
  r.s = mix64(seed ^ mix64(pos + 0x632BE59BD9B4E019ull));
  return r;
}
static inline uint32_t orng_u32(orng* r) {
  r->s += 0x9E3779B97F4A7C15ull;
  return (uint32_t)(mix64(r->s) >> 32);
}
/* uniform in (0,1], like curand_uniform */
static inline float orng_unif(orng* r) { return ((float)(orng_u32(r) >> 8) + 1.0f) * (1.0f / 16777216.0f); }

/* ------------------------------------------------------------------------
 * _GetSubIndptr + exclusive scan: src/cuda/rowwise_sampling.cu:13-40.
 * out_ptr has n+1 entries; returns nnz.
 * ---------------------------------------------------------------------- */
int64_t dgs_oracle_sample_counts(const int64_t* indptr, const int64_t* seeds, int64_t n,
                                 int64_t k, int32_t replace, int64_t* out_ptr) {
  int64_t acc = 0;
  for (int64_t i = 0; i < n; ++i) {
    int64_t deg = indptr[seeds[i] + 1] - indptr[seeds[i]];
    out_ptr[i] = acc;
    acc += replace ? (deg == 0 ? 0 : k) : MIN_(deg, k);
  }
  out_ptr[n] = acc;
  return acc;
}

/* ------------------------------------------------------------------------
 * _CSRRowWiseSampleUniformKernel / ...ReplaceKernel:
 * src/cuda/rowwise_sampling.cu:42-136.
 *  - deg <= k (no replace): copy the row in CSC order (:66-72)  [deterministic]
 *  - else: Algorithm-R reservoir; the reference's atomicMax keeps, per slot,
 *    the largest index that chose it == the serial algorithm's result (:73-96)
 *  - replace: k draws rand % deg (:125-133)
 * pos (optional) receives the picked position inside the row.
 * ---------------------------------------------------------------------- */
void dgs_oracle_sample_uniform(const int64_t* indptr, const int64_t* indices,
                               const int64_t* seeds, int64_t n, int64_t k, int32_t replace,
                               const int64_t* out_ptr, uint64_t rng_seed, int64_t* coo_row,
                               int64_t* coo_col, int64_t* pos) {
#pragma omp parallel
  {
    int64_t* slots = (int64_t*)malloc(sizeof(int64_t) * (size_t)(k > 0 ? k : 1));
#pragma omp for schedule(dynamic, 64)
    for (int64_t i = 0; i < n; ++i) {
      int64_t row = seeds[i];
      int64_t st = indptr[row];
      int64_t deg = indptr[row + 1] - st;
      int64_t o = out_ptr[i];
      orng g = orng_init(rng_seed, (uint64_t)i);
      if (replace) {
        if (deg > 0)
          for (int64_t t = 0; t < k; ++t) {
            int64_t e = (int64_t)(orng_u32(&g) % (uint64_t)deg);
            coo_row[o + t] = row;
            coo_col[o + t] = indices[st + e];
            if (pos) pos[o + t] = e;
          }
      } else if (deg <= k) {
        for (int64_t t = 0; t < deg; ++t) {
          coo_row[o + t] = row;
          coo_col[o + t] = indices[st + t];
          if (pos) pos[o + t] = t;
        }
      } else {
        for (int64_t t = 0; t < k; ++t) slots[t] = t;
        for (int64_t t = k; t < deg; ++t) {
          int64_t num = (int64_t)(orng_u32(&g) % (uint64_t)(t + 1));
          if (num < k) slots[num] = t;
        }
        for (int64_t t = 0; t < k; ++t) {
          coo_row[o + t] = row;
          coo_col[o + t] = indices[st + slots[t]];
          if (pos) pos[o + t] = slots[t];
        }
      }
    }
    free(slots);
  }
}

/* ------------------------------------------------------------------------
 * _CSRRowWiseSampleKernel / ...ReplaceKernel (weighted):
 * src/cuda/rowwise_sampling_probs.cu:54-216.
 *  - deg <= k (no replace): copy the row in order (:123-133)  [deterministic]
 *  - no replace: A-Res key = u^(1/w), keep the k largest, descending (:98-121)
 *  - replace: inclusive prefix of max(w,0); k draws u*sum -> first cdf > draw,
 *    clamped to deg-1 (:175-211)
 * ---------------------------------------------------------------------- */
void dgs_oracle_sample_weighted(const int64_t* indptr, const int64_t* indices,
                                const float* probs, const int64_t* seeds, int64_t n,
                                int64_t k, int32_t replace, const int64_t* out_ptr,
                                uint64_t rng_seed, int64_t* coo_row, int64_t* coo_col,
                                int64_t* pos) {
#pragma omp parallel
  {
    size_t kk = (size_t)(k > 0 ? k : 1);
    float* topk = (float*)malloc(sizeof(float) * kk);
    int64_t* topi = (int64_t*)malloc(sizeof(int64_t) * kk);
    float* cdf = NULL;
    int64_t cdf_cap = 0;
#pragma omp for schedule(dynamic, 64)
    for (int64_t i = 0; i < n; ++i) {
      int64_t row = seeds[i];
      int64_t st = indptr[row];
      int64_t deg = indptr[row + 1] - st;
      int64_t o = out_ptr[i];
      orng g = orng_init(rng_seed, (uint64_t)i);
      if (replace) {
        if (deg <= 0) continue;
        if (deg > cdf_cap) {
          free(cdf);
          cdf_cap = deg * 2;
          cdf = (float*)malloc(sizeof(float) * (size_t)cdf_cap);
        }
        float acc = 0.f;
        for (int64_t t = 0; t < deg; ++t) {
          float w = probs[st + t];
          acc += (w > 0.f ? w : 0.f);
          cdf[t] = acc;
        }
        for (int64_t t = 0; t < k; ++t) {
          float r = orng_unif(&g) * acc;
          int64_t lo = 0, hi = deg; /* upper bound: first cdf[x] > r */
          while (lo < hi) {
            int64_t mid = (lo + hi) >> 1;
            if (cdf[mid] > r) hi = mid; else lo = mid + 1;
          }
          int64_t e = MIN_(lo, deg - 1);
          coo_row[o + t] = row;
          coo_col[o + t] = indices[st + e];
          if (pos) pos[o + t] = e;
        }
      } else if (deg <= k) {
        for (int64_t t = 0; t < deg; ++t) {
          coo_row[o + t] = row;
          coo_col[o + t] = indices[st + t];
          if (pos) pos[o + t] = t;
        }
      } else {
        int64_t cnt = 0;
        for (int64_t t = 0; t < deg; ++t) {
          float key = powf(orng_unif(&g), 1.0f / probs[st + t]);
          /* insertion into a descending list of at most k entries */
          if (cnt < k || key > topk[cnt - 1]) {
            int64_t j = (cnt < k) ? cnt++ : k - 1;
            while (j > 0 && topk[j - 1] < key) {
              topk[j] = topk[j - 1];
              topi[j] = topi[j - 1];
              --j;
            }
            topk[j] = key;
            topi[j] = t;
          }
        }
        for (int64_t t = 0; t < k; ++t) {
          coo_row[o + t] = row;
          coo_col[o + t] = indices[st + topi[t]];
          if (pos) pos[o + t] = topi[t];
        }
      }
    }
    free(topk);
    free(topi);
    free(cdf);
  }
}

/* ------------------------------------------------------------------------
 * Unique + Relabel: src/cuda/tensor_reindex.cu:82-180.
 * The reference stores, per key, the minimum input index (AtomicMin, :28),
 * flags i as "first" iff that minimum equals i (:123), and numbers the flagged
 * entries by an exclusive scan (:125-156): distinct keys in first-occurrence
 * order, independent of hash layout.  Lookup returns the number or -1 (:46-60).
 * The table below is a plain open-addressing map; only the order contract is
 * restated, not the reference's hash function.
 * ---------------------------------------------------------------------- */
typedef struct {
  int64_t* keys;
  int64_t* vals;
  uint64_t mask;
} omap;

static omap omap_new(int64_t n) {
  omap m;
  uint64_t cap = 16;
  while ((int64_t)cap < 2 * n + 2) cap <<= 1;
  m.keys = (int64_t*)malloc(sizeof(int64_t) * cap);
  m.vals = (int64_t*)malloc(sizeof(int64_t) * cap);
  memset(m.keys, 0xFF, sizeof(int64_t) * cap);
  m.mask = cap - 1;
  return m;
}
static inline uint64_t omap_slot(const omap* m, int64_t key, int* found) {
  uint64_t p = mix64((uint64_t)key) & m->mask;
  for (;;) {
    if (m->keys[p] == key) { *found = 1; return p; }
    if (m->keys[p] == -1) { *found = 0; return p; }
    p = (p + 1) & m->mask;
  }
}

/* returns the number of distinct keys written to unique_out (capacity n) */
int64_t dgs_oracle_unique(const int64_t* keys, int64_t n, int64_t* unique_out) {
  omap m = omap_new(n);
  int64_t cnt = 0;
  for (int64_t i = 0; i < n; ++i) {
    int f;
    uint64_t p = omap_slot(&m, keys[i], &f);
    if (!f) {
      m.keys[p] = keys[i];
      m.vals[p] = cnt;
      unique_out[cnt++] = keys[i];
    }
  }
  free(m.keys);
  free(m.vals);
  return cnt;
}

void dgs_oracle_relabel(const int64_t* uniq, int64_t n_unique, const int64_t* in, int64_t n,
                        int64_t* out) {
  omap m = omap_new(n_unique);
  for (int64_t i = 0; i < n_unique; ++i) {
    int f;
    uint64_t p = omap_slot(&m, uniq[i], &f);
    m.keys[p] = uniq[i];
    m.vals[p] = i;
  }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int f;
    uint64_t p = omap_slot(&m, in[i], &f);
    out[i] = f ? m.vals[p] : -1;
  }
  free(m.keys);
  free(m.vals);
}

/* ------------------------------------------------------------------------
 * PaGraph-style cache: src/cuda/pagraph.cu:94-194.  On a hit the row comes
 * from gpu_data[value*D ..], on a miss from cpu_data[nid*D ..].
 * (The table layout is not observable through the fetch result, so the
 * restatement uses a direct key -> value map.)
 * ---------------------------------------------------------------------- */
void dgs_oracle_cache_fetch(const void* cpu_data, const void* gpu_flat, int32_t esz,
                            const int64_t* cache_keys, const int64_t* cache_vals,
                            int64_t n_cache, const int64_t* nid, int64_t n, int64_t D,
                            void* out) {
  omap m = omap_new(n_cache);
  for (int64_t i = 0; i < n_cache; ++i) {
    int f;
    uint64_t p = omap_slot(&m, cache_keys[i], &f);
    m.keys[p] = cache_keys[i];
    m.vals[p] = cache_vals[i];
  }
  size_t rb = (size_t)(D * esz);
  char* o = (char*)out;
  for (int64_t i = 0; i < n; ++i) {
    int f;
    uint64_t p = omap_slot(&m, nid[i], &f);
    if (f) memcpy(o + i * rb, (const char*)gpu_flat + m.vals[p] * rb, rb);
    else memcpy(o + i * rb, (const char*)cpu_data + nid[i] * rb, rb);
  }
  free(m.keys);
  free(m.vals);
}
