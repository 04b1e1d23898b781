// Thread-local error text behind dgs_last_error(); replaces the reference's
// print-and-exit macros (CUDA_CALL / NCCL_CALL / SHM_CHECK,
// src/dgs_headers.h:11-45): failures are returned to the caller as codes.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "../kernels/common.cuh"

namespace dgs {
namespace {
thread_local char g_err[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

// DGS_NO_PDL=1 launches every kernel the plain way (no programmatic stream serialization);
// DGS_PDL_OFF_MASK=<hex> does so for the launch sites whose bit is set
bool chained_launches_enabled(int site) {
  static const unsigned long off = [] {
    const char* e = std::getenv("DGS_NO_PDL");
    if (e != nullptr && e[0] == '1') return ~0ul;
    const char* m = std::getenv("DGS_PDL_OFF_MASK");
    return m != nullptr ? std::strtoul(m, nullptr, 16) : 0ul;
  }();
  return ((off >> site) & 1ul) == 0;
}

int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  set_error("%s:%d: %s failed: %s (%d)", file, line, what, cudaGetErrorString(e), static_cast<int>(e));
  return DGS_ERR_CUDA;
}
}  // namespace dgs

extern "C" const char* dgs_last_error(void) { return dgs::g_err; }

extern "C" int dgs_device_check(void) {
  int dev = 0;
  DGS_CUDA_TRY(cudaGetDevice(&dev));
  cudaDeviceProp prop;
  DGS_CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
  DGS_REQUIRE(prop.major == 10, DGS_ERR_UNSUPPORTED,
              "this library holds sm_100a code only; device %d is sm_%d%d", dev, prop.major, prop.minor);
  return DGS_OK;
}
