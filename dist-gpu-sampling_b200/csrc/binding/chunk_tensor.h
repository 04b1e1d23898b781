// torch.classes.dgs_classes.ChunkTensor: the custom class of the reference
// (src/chunk_tensor.h:61-103, src/chunk_tensor.cc:37-263, registered in
// src/pybind.cc:11-22) as a thin holder of a dgs_store from the C ABI.
#pragma once
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <algorithm>
#include <tuple>
#include <vector>

#include "../../../include/dgs_b200.h"
#include "host_words.h"

namespace dgs {

#define DGS_CHECK_RC(expr)                                                        \
  do {                                                                            \
    int rc__ = (expr);                                                            \
    TORCH_CHECK(rc__ == DGS_OK, "dgs: ", dgs_last_error(), " (code ", rc__, ")"); \
  } while (0)

#define CHECK_CUDA(x) TORCH_CHECK((x).device().is_cuda(), #x " must be a CUDA tensor")

inline cudaStream_t current_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

inline bool is_id64(const torch::Tensor& t, const char* what) {
  TORCH_CHECK(t.scalar_type() == torch::kInt64 || t.scalar_type() == torch::kInt32,
              "ID can only be int32 or int64 (", what, ")");
  return t.scalar_type() == torch::kInt64;
}

inline size_t dtype_size(torch::ScalarType t) {
  // the types ChunkTensor accepts (src/chunk_tensor.cc:15-30)
  switch (t) {
    case torch::kInt32: return 4;
    case torch::kInt64: return 8;
    case torch::kFloat: return 4;
    case torch::kDouble: return 8;
    case torch::kBool: return 1;
    default: TORCH_CHECK(false, "ChunkTensor: unsupported dtype ", t);
  }
}

inline torch::Tensor byte_scratch(size_t bytes, const torch::Device& dev) {
  return torch::empty({static_cast<int64_t>(bytes)}, torch::TensorOptions().dtype(torch::kUInt8).device(dev));
}

class ChunkTensor : public torch::CustomClassHolder {
 public:
  ChunkTensor(std::vector<int64_t> shapes, torch::ScalarType dtype, int64_t capacity_per_gpu) {
    TORCH_CHECK(shapes.size() == 1 || shapes.size() == 2, "ChunkTensor: shape must have 1 or 2 dims");
    TORCH_CHECK(capacity_per_gpu >= 0, "ChunkTensor: capacity_per_gpu must be >= 0");
    dtype_ = dtype;
    const size_t esz = dtype_size(dtype);
    DGS_CHECK_RC(dgs_device_check());
    DGS_CHECK_RC(dgs_store_create(shapes.data(), static_cast<int32_t>(shapes.size()),
                                  static_cast<int32_t>(esz), capacity_per_gpu, &store_));
    DGS_CHECK_RC(dgs_store_desc(store_, &desc_));
    elem_stride_ = dgs_store_elem_stride(store_);
    TORCH_CHECK(cudaGetDevice(&device_) == cudaSuccess, "ChunkTensor: no current CUDA device");
  }
  ~ChunkTensor() override {
    if (store_ != nullptr) dgs_store_destroy(store_);
  }

  torch::Tensor GetHostTensor() {
    void* p = nullptr;
    int64_t n = 0;
    DGS_CHECK_RC(dgs_store_host_view(store_, &p, &n));
    auto opt = torch::TensorOptions().device(torch::kCPU).dtype(dtype_);
    return n > 0 ? torch::from_blob(p, {n}, opt) : torch::empty({0}, opt);
  }

  torch::Tensor GetSubDeviceTensor() {
    void* p = nullptr;
    int64_t n = 0;
    DGS_CHECK_RC(dgs_store_local_view(store_, &p, &n));
    auto opt = torch::TensorOptions().device(torch::Device(torch::kCUDA, device_)).dtype(dtype_);
    return n > 0 ? torch::from_blob(p, {n}, opt) : torch::empty({0}, opt);
  }

  torch::Tensor IndexClass(torch::Tensor index, int32_t location_class, const char* op) {
    CHECK_CUDA(index);
    const bool ids64 = is_id64(index, "index");
    c10::cuda::CUDAGuard guard(index.device());
    const Lease lease(op, index.device().index(), current_stream());
    index = index.contiguous();
    const int64_t n = index.numel();
    torch::Tensor out =
        torch::empty({n, elem_stride_}, torch::TensorOptions().dtype(dtype_).device(index.device()));
    DGS_CHECK_RC(dgs_gather_rows(&desc_, location_class, index.data_ptr(), ids64, n, elem_stride_, out.data_ptr(),
                                 lease.status(), current_stream()));
    lease.finish();
    return out;
  }
  torch::Tensor Index(torch::Tensor index) { return IndexClass(index, DGS_CLASS_ANY, "_CAPI_index"); }
  torch::Tensor LocalIndex(torch::Tensor index) { return IndexClass(index, DGS_CLASS_LOCAL, "_CAPI_local_index"); }
  torch::Tensor RemoteIndex(torch::Tensor index) { return IndexClass(index, DGS_CLASS_REMOTE, "_CAPI_remote_index"); }
  torch::Tensor HostIndex(torch::Tensor index) { return IndexClass(index, DGS_CLASS_HOST, "_CAPI_host_index"); }

  // _CAPI_index with the number of rows taken from the device: out[i] = row index[i] for i < count[0], where
  // `count` is an int64 CUDA tensor written by earlier work on the stream (clamped to index.numel()); the rest
  // of `out` [index.numel(), D] is left as it is.  For callers that queue a gather behind a kernel that
  // produces the ids without reading their number back; the form BlockPipeline uses per batch
  // (dgs_gather_rows_counted).  No counterpart in src/chunk_tensor.h.
  torch::Tensor IndexCounted(torch::Tensor index, torch::Tensor count) {
    CHECK_CUDA(index);
    CHECK_CUDA(count);
    TORCH_CHECK(count.scalar_type() == torch::kInt64 && count.numel() >= 1 && count.device() == index.device(),
                "_CAPI_index_counted: count must be an int64 tensor on the device of index");
    const bool ids64 = is_id64(index, "index");
    c10::cuda::CUDAGuard guard(index.device());
    const Lease lease("_CAPI_index_counted", index.device().index(), current_stream());
    index = index.contiguous();
    const int64_t n = index.numel();
    torch::Tensor out =
        torch::empty({n, elem_stride_}, torch::TensorOptions().dtype(dtype_).device(index.device()));
    DGS_CHECK_RC(dgs_gather_rows_counted(&desc_, index.data_ptr(), ids64, n, count.data_ptr<int64_t>(), elem_stride_,
                                         out.data_ptr(), lease.status(), current_stream()));
    lease.finish();
    return out;
  }

  std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> SplitIndex(torch::Tensor index) {
    CHECK_CUDA(index);
    const bool ids64 = is_id64(index, "index");
    c10::cuda::CUDAGuard guard(index.device());
    const Lease lease("_CAPI_split_index", index.device().index(), current_stream());
    index = index.contiguous().view({-1});
    const int64_t n = index.numel();
    torch::Tensor out = torch::empty_like(index);
    const size_t sb = dgs_split_index_scratch_bytes(n);
    torch::Tensor scratch = byte_scratch(sb, index.device());
    int64_t* counts = lease.sizes();
    DGS_CHECK_RC(dgs_split_index(&desc_, index.data_ptr(), ids64, n, elem_stride_, out.data_ptr(), counts,
                                 scratch.data_ptr(), sb, current_stream()));
    TORCH_CHECK(cudaStreamSynchronize(current_stream()) == cudaSuccess, "dgs: stream synchronisation failed: ",
                cudaGetErrorString(cudaGetLastError()));
    const int64_t nl = counts[0], nr = counts[1], nh = counts[2];
    TORCH_CHECK(nl + nr + nh == n, "dgs: split_index lost ids");
    return std::make_tuple(out.narrow(0, 0, nl), out.narrow(0, nl, nr), out.narrow(0, nl + nr, nh));
  }

  void LoadFromTensor(torch::Tensor data) {
    // argument checks of src/chunk_tensor.cc:174-181
    dgs_chunk_desc d = desc_;
    TORCH_CHECK(data.device().is_cpu(), "_CAPI_load_from_tensor: data must be a CPU tensor");
    TORCH_CHECK(data.scalar_type() == dtype_, "_CAPI_load_from_tensor: dtype mismatch");
    TORCH_CHECK(data.is_contiguous(), "_CAPI_load_from_tensor: data must be contiguous");
    TORCH_CHECK(data.numel() == d.total, "_CAPI_load_from_tensor: shape mismatch");
    TORCH_CHECK(data.dim() == 1 || (data.dim() == 2 && data.size(1) == elem_stride_),
                "_CAPI_load_from_tensor: shape mismatch");
    DGS_CHECK_RC(dgs_store_load(store_, data.data_ptr(), data.numel()));
  }

  const dgs_chunk_desc& desc() const { return desc_; }
  torch::ScalarType dtype() const { return dtype_; }
  int64_t elem_stride() const { return elem_stride_; }
  int device() const { return device_; }

 private:
  dgs_store* store_ = nullptr;
  dgs_chunk_desc desc_;
  torch::ScalarType dtype_;
  int64_t elem_stride_ = 1;
  int device_ = 0;
};

}  // namespace dgs
