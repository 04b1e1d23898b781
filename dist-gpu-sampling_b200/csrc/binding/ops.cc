// PyTorch operator layer: torch.classes.dgs_classes.ChunkTensor and
// torch.ops.dgs_ops.* with the reference's schemas (src/pybind.cc:11-38,
// src/cuda/dgs_ops.h:10-50), implemented as a thin host layer over the C ABI
// of include/dgs_b200.h.  Only this directory (binding/) sees torch types; every
// kernel launch goes through an extern "C" entry point.  chunk_tensor.h holds the
// ChunkTensor class, host_words.h the pinned size / status words leased per call,
// pipeline.h the BlockPipeline class (several mini-batches in flight).
//
// Conventions kept from the reference: one process per GPU, tensors returned
// on the current CUDA device, ChunkTensor construction/destruction collective
// over the communicator set by _CAPI_set_nccl (optional here: without it the
// process is a single-rank group).  Conventions changed: kernels run on
// torch's current stream (the reference uses the legacy default stream, which
// is also torch's default), and every failure surfaces as a c10::Error --
// nothing calls exit()/abort() (src/dgs_headers.h:11-45).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../../include/dgs_b200.h"
#include "chunk_tensor.h"
#include "host_words.h"
#include "pipeline.h"

namespace dgs {
namespace {

dgs_chunk_desc plain_desc(const torch::Tensor& t) {
  dgs_chunk_desc d;
  std::memset(&d, 0, sizeof(d));
  d.total = d.threshold = d.each = t.numel();
  d.num_parts = 1;
  d.local_rank = 0;
  d.esz = static_cast<int32_t>(t.element_size());
  d.dev[0] = t.data_ptr();
  return d;
}

void sync_stream() {
  TORCH_CHECK(cudaStreamSynchronize(current_stream()) == cudaSuccess, "dgs: stream synchronisation failed: ",
              cudaGetErrorString(cudaGetLastError()));
}

}  // namespace

// ===========================================================================
// sampling
// ===========================================================================
namespace {

constexpr int64_t kOneShotOutputBytes = int64_t(1) << 28;  // over-allocate n*k up to 256 MB

std::tuple<torch::Tensor, torch::Tensor> sample_impl(torch::Tensor seeds, const dgs_chunk_desc& indptr,
                                                      torch::ScalarType indptr_dtype,
                                                      const dgs_chunk_desc& indices,
                                                      torch::ScalarType indices_dtype,
                                                      const dgs_chunk_desc* probs, int64_t k, bool replace) {
  CHECK_CUDA(seeds);
  TORCH_CHECK(k >= 0, "num_picks must be >= 0");
  const bool ids64 = is_id64(seeds, "seeds");
  TORCH_CHECK(seeds.scalar_type() == indptr_dtype && seeds.scalar_type() == indices_dtype,
              "seeds, indptr and indices must share one id type");
  c10::cuda::CUDAGuard guard(seeds.device());
  seeds = seeds.contiguous().view({-1});
  const int64_t n = seeds.numel();
  auto opt = seeds.options();
  cudaStream_t stream = current_stream();
  const Lease w("_CAPI_sample_neighbors*", seeds.device().index(), stream);
  const auto rng = next_rng();

  const size_t pb = dgs_sample_plan_bytes(n);
  torch::Tensor plan = byte_scratch(pb, seeds.device());
  const int64_t esz = ids64 ? 8 : 4;
  const bool one_shot = n * k * 2 * esz <= kOneShotOutputBytes;

  auto run = [&](torch::Tensor& row, torch::Tensor& col, int64_t cap, int64_t* nnz) {
    if (probs == nullptr)
      DGS_CHECK_RC(dgs_sample_uniform(&indices, seeds.data_ptr(), ids64, n, k, replace, plan.data_ptr(),
                                      rng.first, rng.second, row.data_ptr(), col.data_ptr(), cap, nnz,
                                      nullptr, w.status(), stream));
    else
      DGS_CHECK_RC(dgs_sample_weighted(&indices, probs, seeds.data_ptr(), ids64, n, k, replace,
                                       plan.data_ptr(), rng.first, rng.second, row.data_ptr(),
                                       col.data_ptr(), cap, nnz, nullptr, w.status(), stream));
  };

  torch::Tensor row, col;
  int64_t nnz = 0;
  if (one_shot) {
    // everything is enqueued first; the host then only waits for the plan
    // kernel's total, not for the sampling kernel behind it
    const int64_t cap = n * k;
    row = torch::empty({cap}, opt);
    col = torch::empty({cap}, opt);
    w.sizes()[0] = kPending;
    DGS_CHECK_RC(dgs_sample_plan(&indptr, seeds.data_ptr(), ids64, n, k, replace, plan.data_ptr(), w.sizes(),
                                 w.status(), stream));
    run(row, col, cap, nullptr);
    nnz = wait_size(w.sizes(), stream, "sample_neighbors");
    if (strict_status()) sync_stream();
    w.check();
    TORCH_CHECK(nnz >= 0 && nnz <= cap, "dgs: sampler returned an impossible size");
    return std::make_tuple(row.narrow(0, 0, nnz), col.narrow(0, 0, nnz));
  }
  DGS_CHECK_RC(dgs_sample_plan(&indptr, seeds.data_ptr(), ids64, n, k, replace, plan.data_ptr(), w.sizes(),
                               w.status(), stream));
  sync_stream();
  nnz = w.sizes()[0];
  w.check();
  row = torch::empty({nnz}, opt);
  col = torch::empty({nnz}, opt);
  run(row, col, nnz, nullptr);
  w.finish();
  return std::make_tuple(row, col);
}

}  // namespace

std::tuple<torch::Tensor, torch::Tensor> RowWiseSamplingUniformCUDA(torch::Tensor seeds, torch::Tensor indptr,
                                                                    torch::Tensor indices,
                                                                    int64_t num_picks, bool replace) {
  CHECK_CUDA(indptr);
  CHECK_CUDA(indices);
  indptr = indptr.contiguous();
  indices = indices.contiguous();
  return sample_impl(seeds, plain_desc(indptr), indptr.scalar_type(), plain_desc(indices),
                     indices.scalar_type(), nullptr, num_picks, replace);
}

std::tuple<torch::Tensor, torch::Tensor> RowWiseSamplingUniformWithChunkTensorCUDA(
    torch::Tensor seeds, c10::intrusive_ptr<ChunkTensor> indptr, c10::intrusive_ptr<ChunkTensor> indices,
    int64_t num_picks, bool replace) {
  return sample_impl(seeds, indptr->desc(), indptr->dtype(), indices->desc(), indices->dtype(), nullptr,
                     num_picks, replace);
}

std::tuple<torch::Tensor, torch::Tensor> RowWiseSamplingProbCUDA(torch::Tensor seeds, torch::Tensor indptr,
                                                                 torch::Tensor indices, torch::Tensor probs,
                                                                 int64_t num_picks, bool replace) {
  CHECK_CUDA(indptr);
  CHECK_CUDA(indices);
  CHECK_CUDA(probs);
  TORCH_CHECK(probs.scalar_type() == torch::kFloat, "probs must be float32");
  indptr = indptr.contiguous();
  indices = indices.contiguous();
  probs = probs.contiguous();
  const dgs_chunk_desc pd = plain_desc(probs);
  return sample_impl(seeds, plain_desc(indptr), indptr.scalar_type(), plain_desc(indices),
                     indices.scalar_type(), &pd, num_picks, replace);
}

std::tuple<torch::Tensor, torch::Tensor> RowWiseSamplingProbWithChunkTensorCUDA(
    torch::Tensor seeds, c10::intrusive_ptr<ChunkTensor> indptr, c10::intrusive_ptr<ChunkTensor> indices,
    c10::intrusive_ptr<ChunkTensor> probs, int64_t num_picks, bool replace) {
  TORCH_CHECK(probs->dtype() == torch::kFloat, "probs must be float32");
  return sample_impl(seeds, indptr->desc(), indptr->dtype(), indices->desc(), indices->dtype(),
                     &probs->desc(), num_picks, replace);
}

// ===========================================================================
// relabel
// ===========================================================================
namespace {
// Up to DGS_MAX_SEGMENTS tensors are passed as a segment list; longer lists
// are concatenated first.  `keep` holds the contiguous tensors alive.
dgs_segments make_segments(const std::vector<torch::Tensor>& ts, std::vector<torch::Tensor>& keep) {
  dgs_segments s;
  std::memset(&s, 0, sizeof(s));
  if (ts.size() > DGS_MAX_SEGMENTS) {
    keep.push_back(torch::cat(ts, 0).contiguous());
    s.count = 1;
    s.ptr[0] = keep.back().data_ptr();
    s.len[0] = keep.back().numel();
    return s;
  }
  s.count = static_cast<int32_t>(ts.size());
  for (size_t i = 0; i < ts.size(); ++i) {
    keep.push_back(ts[i].contiguous());
    s.ptr[i] = keep.back().numel() ? keep.back().data_ptr() : nullptr;
    s.len[i] = keep.back().numel();
  }
  return s;
}
}  // namespace

std::tuple<torch::Tensor, std::vector<torch::Tensor>> TensorRelabelCUDA(
    std::vector<torch::Tensor> mapping_tensors, std::vector<torch::Tensor> requiring_relabel_tensors) {
  TORCH_CHECK(!mapping_tensors.empty(), "_CAPI_tensor_relabel: no mapping tensors");
  const torch::Tensor& first = mapping_tensors[0];
  CHECK_CUDA(first);
  const bool ids64 = is_id64(first, "mapping tensors");
  for (const auto& t : mapping_tensors)
    TORCH_CHECK(t.device() == first.device() && t.scalar_type() == first.scalar_type(),
                "_CAPI_tensor_relabel: all tensors must share device and id type");
  for (const auto& t : requiring_relabel_tensors)
    TORCH_CHECK(t.device() == first.device() && t.scalar_type() == first.scalar_type(),
                "_CAPI_tensor_relabel: all tensors must share device and id type");
  c10::cuda::CUDAGuard guard(first.device());
  cudaStream_t stream = current_stream();
  const Lease w("_CAPI_tensor_relabel", first.device().index(), stream);

  std::vector<torch::Tensor> keep;
  const dgs_segments keys = make_segments(mapping_tensors, keep);
  int64_t n_keys = 0;
  for (int i = 0; i < keys.count; ++i) n_keys += keys.len[i];
  const dgs_segments req = make_segments(requiring_relabel_tensors, keep);
  int64_t n_req = 0;
  std::vector<int64_t> split_sizes;
  for (const auto& t : requiring_relabel_tensors) {
    split_sizes.push_back(t.numel());
    n_req += t.numel();
  }

  const size_t tb = dgs_relabel_table_bytes(n_keys);
  torch::Tensor table = byte_scratch(tb, first.device());
  torch::Tensor uniq = torch::empty({n_keys}, first.options());
  torch::Tensor out = torch::empty({n_req}, first.options());
  // the count kernel reports the number of distinct keys; the numbering and
  // lookup kernels behind it are still in flight when this returns
  w.sizes()[0] = kPending;
  DGS_CHECK_RC(dgs_unique_first_occurrence(&keys, ids64, table.data_ptr(), tb, uniq.data_ptr(), w.sizes(),
                                           w.status(), stream));
  DGS_CHECK_RC(dgs_relabel_lookup(table.data_ptr(), tb, n_keys, &req, ids64, out.data_ptr(), stream));
  const int64_t nu = wait_size(w.sizes(), stream, "_CAPI_tensor_relabel");
  if (strict_status()) sync_stream();
  w.check();
  TORCH_CHECK(nu >= 0 && nu <= n_keys, "dgs: relabel returned an impossible size");
  return std::make_tuple(uniq.narrow(0, 0, nu), out.split_with_sizes(split_sizes, 0));
}

// ===========================================================================
// multi-hop sample + relabel in one queued sequence
// ===========================================================================
namespace {

using BlocksResult =
    std::tuple<torch::Tensor, std::vector<torch::Tensor>, std::vector<torch::Tensor>, std::vector<int64_t>>;

// workspace + outputs the one-sequence path may hold (they are sized by upper
// bounds, not by what the hops turn out to need); larger requests go hop by hop
constexpr int64_t kBlocksBudgetBytes = int64_t(2) << 30;

BlocksResult blocks_impl(torch::Tensor seeds, const dgs_chunk_desc& indptr, torch::ScalarType indptr_dtype,
                         const dgs_chunk_desc& indices, torch::ScalarType indices_dtype,
                         const dgs_chunk_desc* probs, const std::vector<int64_t>& fanouts, bool replace) {
  CHECK_CUDA(seeds);
  const bool ids64 = is_id64(seeds, "seeds");
  TORCH_CHECK(seeds.scalar_type() == indptr_dtype && seeds.scalar_type() == indices_dtype,
              "seeds, indptr and indices must share one id type");
  const int H = static_cast<int>(fanouts.size());
  TORCH_CHECK(H >= 1, "sample_blocks: no fan-outs");
  for (int64_t k : fanouts) TORCH_CHECK(k >= 0, "num_picks must be >= 0");
  c10::cuda::CUDAGuard guard(seeds.device());
  seeds = seeds.contiguous().view({-1});
  const int64_t n = seeds.numel();
  const int64_t esz = ids64 ? 8 : 4;
  // the reference applies the fan-outs last to first (chunktensor_sampler.py:97)
  std::vector<int64_t> applied(fanouts.rbegin(), fanouts.rend());

  std::vector<torch::Tensor> rows(H), cols(H);
  std::vector<int64_t> shape(2 * H);
  torch::Tensor frontier;

  dgs_hop hops[DGS_MAX_HOPS];
  bool sequence = n > 0 && H <= DGS_MAX_HOPS;
  for (int64_t k : applied) sequence = sequence && k >= 1;
  if (sequence) sequence = dgs_sample_blocks_bounds(n, applied.data(), H, indptr.total - 1, hops) == DGS_OK;
  size_t ws_bytes = 0;
  if (sequence) {
    ws_bytes = dgs_sample_blocks_workspace_bytes(hops, H);
    int64_t total = static_cast<int64_t>(ws_bytes);
    for (int h = 0; h < H; ++h) total += (2 * hops[h].seed_bound * hops[h].fanout + hops[h].frontier_bound) * esz;
    sequence = total <= kBlocksBudgetBytes;
  }

  // hop by hop through the per-operator path: empty input, zero fan-outs, very large bounds, or a frontier
  // that outgrew the bound of the one-sequence path (see below)
  auto hop_by_hop = [&]() -> BlocksResult {
    torch::Tensor cur = seeds;
    for (int h = 0; h < H; ++h) {
      auto rc = sample_impl(cur, indptr, indptr_dtype, indices, indices_dtype, probs, applied[h], replace);
      auto rl = TensorRelabelCUDA({cur, std::get<1>(rc)}, {std::get<0>(rc), std::get<1>(rc)});
      const int at = H - 1 - h;
      rows[at] = std::get<1>(rl)[0];
      cols[at] = std::get<1>(rl)[1];
      shape[2 * at] = std::get<0>(rl).numel();
      shape[2 * at + 1] = cur.numel();
      cur = std::get<0>(rl);
    }
    return std::make_tuple(cur, rows, cols, shape);
  };
  if (!sequence) return hop_by_hop();

  auto opt = seeds.options();
  cudaStream_t stream = current_stream();
  const Lease w("_CAPI_sample_blocks*", seeds.device().index(), stream);
  const auto rng = next_rng(static_cast<uint64_t>(H));
  torch::Tensor ws = byte_scratch(ws_bytes, seeds.device());
  std::vector<torch::Tensor> fr(H);
  for (int h = 0; h < H; ++h) {
    const int64_t cap = hops[h].seed_bound * hops[h].fanout;
    rows[H - 1 - h] = torch::empty({cap}, opt);
    cols[H - 1 - h] = torch::empty({cap}, opt);
    fr[h] = torch::empty({hops[h].frontier_bound}, opt);
    hops[h].coo_row = rows[H - 1 - h].data_ptr();
    hops[h].coo_col = cols[H - 1 - h].data_ptr();
    hops[h].frontier = fr[h].data_ptr();
    w.sizes()[2 * h] = w.sizes()[2 * h + 1] = kPending;
  }
  DGS_CHECK_RC(dgs_sample_blocks(&indptr, &indices, probs, seeds.data_ptr(), ids64, hops, H, replace, rng.first,
                                 rng.second, ws.data_ptr(), ws_bytes, w.sizes(), w.status(), stream));
  // the one read-back: the last size lands while that hop's numbering and lookup still run
  int64_t n_dst = n;
  bool outgrown = false;
  for (int h = 0; h < H; ++h) {
    const int64_t nnz = wait_size(w.sizes() + 2 * h, stream, "sample_blocks");
    const int64_t nu = wait_size(w.sizes() + 2 * h + 1, stream, "sample_blocks");
    TORCH_CHECK(nnz >= 0 && nnz <= hops[h].seed_bound * hops[h].fanout && nu >= 0,
                "dgs: sample_blocks returned an impossible size");
    outgrown = outgrown || nu > hops[h].frontier_bound;
  }
  if (outgrown) {
    // The bound assumes that neighbour ids lie in indptr's node space.  On a bipartite CSC whose column ids
    // live in a larger space a hop can find more distinct ids than indptr has rows; the per-hop operators have
    // no such assumption, so the batch is run again through them.  The out-of-range status the numbering
    // kernel raised for the cut-off frontier belongs to the bound, not to the caller's input.
    sync_stream();
    if (*w.status() == DGS_ERR_RANGE) *w.status() = 0;
    w.check();
    for (int h = 0; h < H; ++h) rows[h] = cols[h] = torch::Tensor();
    return hop_by_hop();
  }
  for (int h = 0; h < H; ++h) {
    const int64_t nnz = w.sizes()[2 * h], nu = w.sizes()[2 * h + 1];
    const int at = H - 1 - h;
    rows[at] = rows[at].narrow(0, 0, nnz);
    cols[at] = cols[at].narrow(0, 0, nnz);
    shape[2 * at] = std::min(nu, hops[h].frontier_bound);
    shape[2 * at + 1] = n_dst;
    n_dst = shape[2 * at];
  }
  if (strict_status()) sync_stream();
  w.check();
  frontier = fr[H - 1].narrow(0, 0, n_dst);
  return std::make_tuple(frontier, rows, cols, shape);
}

}  // namespace

// (frontier, coo_rows, coo_cols, [n_src_0, n_dst_0, n_src_1, n_dst_1, ...]) with the blocks in layer
// order, outermost hop first, as ChunkTensorSampler.sample_blocks builds its list
BlocksResult SampleBlocksCUDA(torch::Tensor seeds, torch::Tensor indptr, torch::Tensor indices,
                              std::vector<int64_t> fanouts, bool replace) {
  CHECK_CUDA(indptr);
  CHECK_CUDA(indices);
  indptr = indptr.contiguous();
  indices = indices.contiguous();
  return blocks_impl(seeds, plain_desc(indptr), indptr.scalar_type(), plain_desc(indices), indices.scalar_type(),
                     nullptr, fanouts, replace);
}

BlocksResult SampleBlocksWithChunkTensorCUDA(torch::Tensor seeds, c10::intrusive_ptr<ChunkTensor> indptr,
                                             c10::intrusive_ptr<ChunkTensor> indices, std::vector<int64_t> fanouts,
                                             bool replace) {
  return blocks_impl(seeds, indptr->desc(), indptr->dtype(), indices->desc(), indices->dtype(), nullptr, fanouts,
                     replace);
}

BlocksResult SampleBlocksProbCUDA(torch::Tensor seeds, torch::Tensor indptr, torch::Tensor indices,
                                  torch::Tensor probs, std::vector<int64_t> fanouts, bool replace) {
  CHECK_CUDA(indptr);
  CHECK_CUDA(indices);
  CHECK_CUDA(probs);
  TORCH_CHECK(probs.scalar_type() == torch::kFloat, "probs must be float32");
  indptr = indptr.contiguous();
  indices = indices.contiguous();
  probs = probs.contiguous();
  const dgs_chunk_desc pd = plain_desc(probs);
  return blocks_impl(seeds, plain_desc(indptr), indptr.scalar_type(), plain_desc(indices), indices.scalar_type(),
                     &pd, fanouts, replace);
}

BlocksResult SampleBlocksProbWithChunkTensorCUDA(torch::Tensor seeds, c10::intrusive_ptr<ChunkTensor> indptr,
                                                 c10::intrusive_ptr<ChunkTensor> indices,
                                                 c10::intrusive_ptr<ChunkTensor> probs, std::vector<int64_t> fanouts,
                                                 bool replace) {
  TORCH_CHECK(probs->dtype() == torch::kFloat, "probs must be float32");
  return blocks_impl(seeds, indptr->desc(), indptr->dtype(), indices->desc(), indices->dtype(), &probs->desc(),
                     fanouts, replace);
}

// ===========================================================================
// PaGraph-style cache
// ===========================================================================
std::tuple<torch::Tensor, torch::Tensor> CreateHashMapTensorCUDA(torch::Tensor input_key,
                                                                 torch::Tensor input_value) {
  CHECK_CUDA(input_key);
  CHECK_CUDA(input_value);
  const bool ids64 = is_id64(input_key, "input_key");
  TORCH_CHECK(input_value.scalar_type() == input_key.scalar_type(), "key and value must share one id type");
  TORCH_CHECK(input_value.numel() == input_key.numel(), "key and value must have the same length");
  c10::cuda::CUDAGuard guard(input_key.device());
  input_key = input_key.contiguous();
  input_value = input_value.contiguous();
  const int64_t n = input_key.numel();
  const int64_t slots = dgs_cache_table_slots(n);
  torch::Tensor kb = torch::empty({slots}, input_key.options());
  torch::Tensor vb = torch::empty({slots}, input_value.options());
  const Lease w("_CAPI_create_hash_map", input_key.device().index(), current_stream());
  DGS_CHECK_RC(dgs_cache_build(input_key.data_ptr(), input_value.data_ptr(), ids64, n, kb.data_ptr(),
                               vb.data_ptr(), slots, w.status(), current_stream()));
  w.finish();
  return std::make_tuple(kb, vb);
}

namespace {
torch::Tensor fetch_impl(torch::Tensor cpu_data, const dgs_chunk_desc& gpu, torch::ScalarType gpu_dtype,
                         torch::Tensor nid, torch::Tensor hk, torch::Tensor hv) {
  CHECK_CUDA(nid);
  CHECK_CUDA(hk);
  CHECK_CUDA(hv);
  TORCH_CHECK(cpu_data.dim() == 2 && cpu_data.is_contiguous(), "cpu_data must be a contiguous 2-D tensor");
  TORCH_CHECK(cpu_data.is_cuda() || cpu_data.is_pinned(),
              "cpu_data must be pinned (page-locked) so that the GPU can read it in place");
  TORCH_CHECK(cpu_data.scalar_type() == gpu_dtype, "cpu_data and gpu_data must share one dtype");
  const bool ids64 = is_id64(nid, "nid");
  TORCH_CHECK(hk.scalar_type() == nid.scalar_type() && hv.scalar_type() == nid.scalar_type(),
              "nid and the hash tensors must share one id type");
  c10::cuda::CUDAGuard guard(nid.device());
  nid = nid.contiguous();
  const int64_t n = nid.numel(), D = cpu_data.size(1);
  torch::Tensor out = torch::empty({n, D}, torch::TensorOptions().dtype(gpu_dtype).device(nid.device()));
  const Lease w("_CAPI_fetch_data*", nid.device().index(), current_stream());
  DGS_CHECK_RC(dgs_cache_fetch(cpu_data.data_ptr(), cpu_data.size(0), &gpu, nid.data_ptr(), ids64, n, D,
                               hk.data_ptr(), hv.data_ptr(), hk.numel(), out.data_ptr(), w.status(),
                               current_stream()));
  w.finish();
  return out;
}
}  // namespace

torch::Tensor FetchDataCUDA(torch::Tensor cpu_data, torch::Tensor gpu_data, torch::Tensor nid,
                            torch::Tensor hashed_key_tensor, torch::Tensor hashed_value_tensor) {
  CHECK_CUDA(gpu_data);
  gpu_data = gpu_data.contiguous();
  return fetch_impl(cpu_data, plain_desc(gpu_data), gpu_data.scalar_type(), nid, hashed_key_tensor,
                    hashed_value_tensor);
}

torch::Tensor FetchDataWithChunkTensorCUDA(torch::Tensor cpu_data, c10::intrusive_ptr<ChunkTensor> gpu_data,
                                           torch::Tensor nid, torch::Tensor hashed_key_tensor,
                                           torch::Tensor hashed_value_tensor) {
  return fetch_impl(cpu_data, gpu_data->desc(), gpu_data->dtype(), nid, hashed_key_tensor,
                    hashed_value_tensor);
}

// ===========================================================================
// communicator + bookkeeping
// ===========================================================================
std::vector<int64_t> GetUniqueId() {
  std::vector<int64_t> id(16);
  DGS_CHECK_RC(dgs_comm_get_unique_id(id.data()));
  return id;
}

void SetNCCL(int64_t nranks, std::vector<int64_t> unique_id_array, int64_t rank) {
  TORCH_CHECK(unique_id_array.size() >= 16, "_CAPI_set_nccl: unique id must hold 16 int64");
  DGS_CHECK_RC(dgs_comm_init(nranks, unique_id_array.data(), rank));
}

int64_t GetCurrAllocated() { return dgs_alloc_current_bytes(); }

}  // namespace dgs

using namespace dgs;

TORCH_LIBRARY(dgs_classes, m) {
  m.class_<ChunkTensor>("ChunkTensor")
      .def(torch::init<std::vector<int64_t>, torch::ScalarType, int64_t>())
      .def("_CAPI_get_host_tensor", &ChunkTensor::GetHostTensor)
      .def("_CAPI_get_sub_device_tensor", &ChunkTensor::GetSubDeviceTensor)
      .def("_CAPI_index", &ChunkTensor::Index)
      .def("_CAPI_split_index", &ChunkTensor::SplitIndex)
      .def("_CAPI_local_index", &ChunkTensor::LocalIndex)
      .def("_CAPI_remote_index", &ChunkTensor::RemoteIndex)
      .def("_CAPI_host_index", &ChunkTensor::HostIndex)
      .def("_CAPI_load_from_tensor", &ChunkTensor::LoadFromTensor)
      // addition (no counterpart in src/pybind.cc): the gather with its row count on the device
      .def("_CAPI_index_counted", &ChunkTensor::IndexCounted);
  // addition (no counterpart in src/pybind.cc): mini-batches in flight, see pipeline.h
  m.class_<BlockPipeline>("BlockPipeline")
      .def(torch::init<c10::intrusive_ptr<ChunkTensor>, c10::intrusive_ptr<ChunkTensor>,
                       c10::optional<c10::intrusive_ptr<ChunkTensor>>, c10::optional<c10::intrusive_ptr<ChunkTensor>>,
                       std::vector<int64_t>, bool, int64_t, int64_t, int64_t>())
      .def("submit", &BlockPipeline::submit)
      .def("next", &BlockPipeline::next)
      .def("pending", &BlockPipeline::pending)
      .def("recorded_slots", &BlockPipeline::recorded_slots)
      .def("depth", &BlockPipeline::depth);
}

TORCH_LIBRARY(dgs_ops, m) {
  m.def("_CAPI_tensor_relabel", &TensorRelabelCUDA)
      .def("_CAPI_sample_neighbors", &RowWiseSamplingUniformCUDA)
      .def("_CAPI_sample_neighbors_with_chunk_tensor", &RowWiseSamplingUniformWithChunkTensorCUDA)
      .def("_CAPI_sample_neighbors_with_probs", &RowWiseSamplingProbCUDA)
      .def("_CAPI_sample_neighbors_with_probs_with_chunk_tensor", &RowWiseSamplingProbWithChunkTensorCUDA)
      .def("_CAPI_sample_blocks", &SampleBlocksCUDA)
      .def("_CAPI_sample_blocks_with_chunk_tensor", &SampleBlocksWithChunkTensorCUDA)
      .def("_CAPI_sample_blocks_with_probs", &SampleBlocksProbCUDA)
      .def("_CAPI_sample_blocks_with_probs_with_chunk_tensor", &SampleBlocksProbWithChunkTensorCUDA)
      .def("_CAPI_create_hash_map", &CreateHashMapTensorCUDA)
      .def("_CAPI_fetch_data", &FetchDataCUDA)
      .def("_CAPI_fetch_data_chunk_tensor", &FetchDataWithChunkTensorCUDA)
      .def("_CAPI_get_unique_id", &GetUniqueId)
      .def("_CAPI_set_nccl", &SetNCCL)
      .def("_CAPI_get_current_allocated", &GetCurrAllocated);
}
