// KV-cache write side: scatter new K/V rows into the pages of a paged cache.
//
// The paged decode kernels read token t of sequence b at
//     pool[block_table[b, t / page_size], t % page_size, kv head, :]
// (the two-level load of the reference, loopfuse/codegen.py:738-872, over the cache layout of
// its benchmark, tests/benchmark.py:308-319). This kernel is the producer of that format on the
// device: the same index arithmetic, used as a store address. It is pure data movement, bound by
// HBM bandwidth for a prefill-sized append and by launch latency for a one-token append.
#include "lf_common.cuh"

namespace lf {

struct KvAppendParams {
  const __nv_bfloat16* k_new;
  const __nv_bfloat16* v_new;
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;
  const int32_t* block_table;
  const int32_t* block_table_v;
  const int32_t* seq_pos;
  int32_t start_pos;
  int32_t B, Hkv, T;
  int64_t kn_stride[3], vn_stride[3];
  int64_t kp_stride[3], vp_stride[3];
  int64_t bt_stride;
  int32_t bt_blocks, page_size, page_shift, n_pages;
  int32_t* status;
};

// One thread moves one 16-byte piece of a K row and the same piece of the V row. Consecutive
// threads take consecutive pieces of a row, then consecutive tokens, so a warp reads and writes
// whole 256-byte (D = 128) rows.
template <int D>
__global__ void __launch_bounds__(256) kv_append_kernel(const KvAppendParams p) {
  constexpr int CPR = D / 8;  // 16-byte pieces per row
  const int64_t total = static_cast<int64_t>(p.B) * p.Hkv * p.T * CPR;
  for (int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < total;
       gid += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(gid % CPR);
    const int64_t row = gid / CPR;
    const int t = static_cast<int>(row % p.T);
    const int h = static_cast<int>((row / p.T) % p.Hkv);
    const int b = static_cast<int>(row / p.T / p.Hkv);
    const int pos = (p.seq_pos ? p.seq_pos[b] : p.start_pos) + t;
    const int blk = p.page_shift >= 0 ? (pos >> p.page_shift) : (pos / p.page_size);
    const int slot = pos - blk * p.page_size;
    if (pos < 0 || blk >= p.bt_blocks) {  // the table has no page for this position
      if (p.status) atomicExch(p.status, LF_DEV_BAD_PAGE);
      continue;
    }
    const int32_t pk = p.block_table[b * p.bt_stride + blk];
    const int32_t pv = p.block_table_v[b * p.bt_stride + blk];
    if (pk < 0 || pk >= p.n_pages || pv < 0 || pv >= p.n_pages) {  // never write outside the pool
      if (p.status) atomicExch(p.status, LF_DEV_BAD_PAGE);
      continue;
    }
    if (!LF_BOUNDS(b < p.B && h < p.Hkv && t < p.T && c < CPR && slot >= 0 && slot < p.page_size,
                   p.status, 50))
      continue;
    const uint4 kx = ldg_stream_16(p.k_new + b * p.kn_stride[0] + h * p.kn_stride[1] +
                                   static_cast<int64_t>(t) * p.kn_stride[2] + c * 8);
    const uint4 vx = ldg_stream_16(p.v_new + b * p.vn_stride[0] + h * p.vn_stride[1] +
                                   static_cast<int64_t>(t) * p.vn_stride[2] + c * 8);
    *reinterpret_cast<uint4*>(p.k_pool + pk * p.kp_stride[0] + slot * p.kp_stride[1] +
                              h * p.kp_stride[2] + c * 8) = kx;
    *reinterpret_cast<uint4*>(p.v_pool + pv * p.vp_stride[0] + slot * p.vp_stride[1] +
                              h * p.vp_stride[2] + c * 8) = vx;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace lf

extern "C" int lf_kv_append_bf16(const LfKvAppendArgs* a, void* stream) {
  using namespace lf;
  if (!a || !a->k_new || !a->v_new || !a->k_pool || !a->v_pool || !a->block_table)
    return LF_ERR_INVALID_ARG;
  if (a->B <= 0 || a->Hkv <= 0 || a->T <= 0 || a->page_size <= 0 || a->n_pages <= 0 ||
      a->bt_blocks <= 0)
    return LF_ERR_INVALID_ARG;
  if (a->D != 64 && a->D != 128) return LF_ERR_UNSUPPORTED;
  if (!a->seq_pos && a->start_pos < 0) return LF_ERR_INVALID_ARG;
  if (!aligned16(a->k_new) || !aligned16(a->v_new) || !aligned16(a->k_pool) ||
      !aligned16(a->v_pool))
    return LF_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if ((a->kn_stride[i] % 8) || (a->vn_stride[i] % 8) || (a->kp_stride[i] % 8) ||
        (a->vp_stride[i] % 8))
      return LF_ERR_ALIGNMENT;

  KvAppendParams p;
  p.k_new = static_cast<const __nv_bfloat16*>(a->k_new);
  p.v_new = static_cast<const __nv_bfloat16*>(a->v_new);
  p.k_pool = static_cast<__nv_bfloat16*>(a->k_pool);
  p.v_pool = static_cast<__nv_bfloat16*>(a->v_pool);
  p.block_table = a->block_table;
  p.block_table_v = a->block_table_v ? a->block_table_v : a->block_table;
  p.seq_pos = a->seq_pos;
  p.start_pos = a->start_pos;
  p.B = a->B;
  p.Hkv = a->Hkv;
  p.T = a->T;
  for (int i = 0; i < 3; ++i) {
    p.kn_stride[i] = a->kn_stride[i];
    p.vn_stride[i] = a->vn_stride[i];
    p.kp_stride[i] = a->kp_stride[i];
    p.vp_stride[i] = a->vp_stride[i];
  }
  p.bt_stride = a->bt_stride;
  p.bt_blocks = a->bt_blocks;
  p.page_size = a->page_size;
  p.page_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == a->page_size) p.page_shift = sh;
  p.n_pages = a->n_pages;
  p.status = a->status;

  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t total = static_cast<int64_t>(a->B) * a->Hkv * a->T * (a->D / 8);
  // Small appends get just the CTAs they need; large ones a grid of 32 CTAs per SM (a multiple
  // of the SM count) that strides over the rest.
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sms) * 32;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->D == 128)
    kv_append_kernel<128><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p);
  else
    kv_append_kernel<64><<<static_cast<unsigned>(blocks), 256, 0, st>>>(p);
  return check_launch("kv_append_kernel");
}
