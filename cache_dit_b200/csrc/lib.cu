// Library-wide plumbing of the C ABI: version, status text, error capture, device queries.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace cdb {

static thread_local char g_cuda_error[512] = "";

void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", cudaGetErrorName(e),
           cudaGetErrorString(e), where ? where : "?");
}

void set_error_text(const char* text) { snprintf(g_cuda_error, sizeof(g_cuda_error), "%s", text ? text : ""); }

bool pdl_enabled() {
  static const bool on = [] {
    const char* env = getenv("CDB_PDL");
    return !(env && env[0] == '0');
  }();
  return on;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace cdb

extern "C" int cdb_abi_version(void) { return 1; }

extern "C" const char* cdb_status_string(int status) {
  switch (status) {
    case CDB_OK: return "ok";
    case CDB_ERR_BAD_ARGUMENT: return "bad argument";
    case CDB_ERR_UNSUPPORTED: return "unsupported shape or alignment";
    case CDB_ERR_SCRATCH_TOO_SMALL: return "scratch buffer too small";
    case CDB_ERR_CUDA: return "CUDA call failed";
    case CDB_ERR_NO_DEVICE: return "no sm_100 device";
    case CDB_ERR_DEVICE_TIMEOUT: return "bounded device-side wait expired";
    case CDB_ERR_TOO_LARGE: return "size exceeds the limit of this entry point";
    default: return "unknown status";
  }
}

extern "C" const char* cdb_last_cuda_error(void) { return cdb::g_cuda_error; }
