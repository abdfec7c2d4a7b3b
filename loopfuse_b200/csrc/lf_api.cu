// Library-wide pieces of the C ABI: error text, device query, launch checking.
#include "lf_common.cuh"

#include <stdio.h>
#include <string.h>

namespace lf {

static thread_local char g_cuda_error[256] = "";

void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e),
           cudaGetErrorString(e));
}

// Launch errors only (no synchronisation): the launch stays asynchronous.
int check_launch(const char* where) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return LF_OK;
  set_cuda_error(e, where);
  return LF_ERR_CUDA;
}

}  // namespace lf

extern "C" {

const char* lf_strerror(int status) {
  switch (status) {
    case LF_OK: return "ok";
    case LF_ERR_INVALID_ARG: return "invalid argument";
    case LF_ERR_UNSUPPORTED: return "unsupported configuration (no kernel for it)";
    case LF_ERR_ALIGNMENT: return "pointer or stride not aligned to 16 bytes";
    case LF_ERR_WORKSPACE: return "split-KV workspace missing or too small";
    case LF_ERR_CUDA: return "CUDA call failed (see lf_last_cuda_error)";
    case LF_ERR_NO_DEVICE: return "no sm_100 CUDA device is current";
    case LF_ERR_TOO_LARGE: return "size beyond the limit of this entry point";
    default: return "unknown status";
  }
}

const char* lf_last_cuda_error(void) { return lf::g_cuda_error; }

int lf_query(LfDeviceInfo* info) {
  if (!info) return LF_ERR_INVALID_ARG;
  memset(info, 0, sizeof(*info));
  info->abi_version = LF_ABI_VERSION;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    lf::set_cuda_error(e, "cudaGetDevice");
    cudaGetLastError();
    return LF_ERR_NO_DEVICE;
  }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) {
    lf::set_cuda_error(e, "cudaGetDeviceProperties");
    cudaGetLastError();
    return LF_ERR_NO_DEVICE;
  }
  info->device = dev;
  info->cc_major = prop.major;
  info->cc_minor = prop.minor;
  info->sm_count = prop.multiProcessorCount;
  info->max_smem_optin = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
  info->total_mem = static_cast<int64_t>(prop.totalGlobalMem);
  return prop.major == 10 ? LF_OK : LF_ERR_NO_DEVICE;
}

}  // extern "C"
