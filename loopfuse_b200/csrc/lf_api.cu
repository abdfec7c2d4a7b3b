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

// Self-test of the bounded device-side wait: one thread waits, with a caller-given short limit,
// on an mbarrier that nobody ever arrives on. The wait runs out, the kernel records
// LF_DEV_TIMEOUT | (site 99 << 8) in the status word and returns normally - the same way every
// kernel of the library reacts to a wait that does not complete (nothing traps, nothing spins
// for ever, the context stays usable).
__global__ void selftest_wait_kernel(long long limit_cycles, int32_t* status, long long* waited) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    const long long t0 = clock64();
    const bool ok = mbar_wait(&bar, 0, limit_cycles);
    if (waited) *waited = clock64() - t0;
    if (!ok && status) atomicCAS(status, LF_DEV_OK, LF_DEV_TIMEOUT | (99 << 8));
  }
}

}  // namespace lf

extern "C" {

int lf_debug_bounds(void) {
#ifdef LF_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}

int lf_selftest_wait_timeout(int64_t limit_cycles, int32_t* status, int64_t* waited_cycles,
                             void* stream) {
  if (limit_cycles <= 0 || limit_cycles > 2000000000ll || !status) return LF_ERR_INVALID_ARG;
  lf::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      limit_cycles, status, reinterpret_cast<long long*>(waited_cycles));
  return lf::check_launch("selftest_wait_kernel");
}

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
