// Elementwise bf16 add on [B, H, S, D] tensors: the query bias (Q + q_bias, before the attention
// kernel) and the output bias (scores @ V + out_bias, after it) of the reference's modified
// attention (tests/test_accuracy.py:176-194; the reference fuses both into its generated kernel,
// loopfuse/codegen.py:454-998). Each is one rounding to bf16, exactly what the eager graph does,
// so a separate pass gives the same bits as a fused one would; both are HBM-bound and small next
// to the attention itself (the additive *score* bias, which is as large as the score matrix, is
// read inside the attention kernel instead).
#include "lf_common.cuh"

namespace lf {

struct AddParams {
  const __nv_bfloat16* a;
  const __nv_bfloat16* b;
  __nv_bfloat16* out;
  int32_t H, S, cpr;  // cpr = 16-byte pieces per row
  int64_t total;      // pieces in all
  int64_t as[3], bs[3], os[3];
};

__device__ __forceinline__ uint32_t add_bf16x2(uint32_t x, uint32_t y) {
  const float lo = __uint_as_float(x << 16) + __uint_as_float(y << 16);
  const float hi = __uint_as_float(x & 0xffff0000u) + __uint_as_float(y & 0xffff0000u);
  return pack_bf16x2(lo, hi);
}

// One thread adds one 16-byte piece; consecutive threads take consecutive pieces of a row.
__global__ void __launch_bounds__(256) add_bf16_kernel(const AddParams p) {
  for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < p.total;
       gid += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(gid % p.cpr);
    int64_t row = gid / p.cpr;
    const int s = static_cast<int>(row % p.S);
    row /= p.S;
    const int h = static_cast<int>(row % p.H);
    const int64_t b = row / p.H;
    const uint4 x = *reinterpret_cast<const uint4*>(p.a + b * p.as[0] + h * p.as[1] + s * p.as[2] + c * 8);
    const uint4 y = ldg_stream_16(p.b + b * p.bs[0] + h * p.bs[1] + s * p.bs[2] + c * 8);
    uint4 r;
    r.x = add_bf16x2(x.x, y.x);
    r.y = add_bf16x2(x.y, y.y);
    r.z = add_bf16x2(x.z, y.z);
    r.w = add_bf16x2(x.w, y.w);
    *reinterpret_cast<uint4*>(p.out + b * p.os[0] + h * p.os[1] + s * p.os[2] + c * 8) = r;
  }
}

}  // namespace lf

extern "C" int lf_add_bf16(const void* a, const void* b, void* out, int32_t B, int32_t H,
                           int32_t S, int32_t D, const int64_t* a_stride,
                           const int64_t* b_stride, const int64_t* out_stride, void* stream) {
  using namespace lf;
  if (!a || !b || !out || !a_stride || !b_stride || !out_stride) return LF_ERR_INVALID_ARG;
  if (B <= 0 || H <= 0 || S <= 0 || D <= 0 || D % 8) return LF_ERR_INVALID_ARG;
  const void* ptrs[3] = {a, b, out};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15u) return LF_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if (a_stride[i] % 8 || b_stride[i] % 8 || out_stride[i] % 8) return LF_ERR_ALIGNMENT;
  AddParams p;
  p.a = static_cast<const __nv_bfloat16*>(a);
  p.b = static_cast<const __nv_bfloat16*>(b);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.H = H;
  p.S = S;
  p.cpr = D / 8;
  p.total = static_cast<int64_t>(B) * H * S * p.cpr;
  for (int i = 0; i < 3; ++i) {
    p.as[i] = a_stride[i];
    p.bs[i] = b_stride[i];
    p.os[i] = out_stride[i];
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t blocks = (p.total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sms) * 32;  // a multiple of the SM count
  if (blocks > cap) blocks = cap;
  add_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch("add_bf16_kernel");
}
