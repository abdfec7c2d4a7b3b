// Prefill attention for sm_100a: TMA-staged tiles, tcgen05 MMA with accumulators in tensor
// memory, online softmax in registers. Two kernels share the tile shapes, the shared-memory
// and tensor-memory layouts and the host code of this file:
//
//   prefill_kernel<D, MODE> (this file): the running-max modes - plain scores, generic score
//       mods, softcap with a large cap. One CTA per pair of query tiles.
//   prefill_bounded_kernel<D> (lf_prefill_bounded.cuh): softcap whose output range needs no
//       running max (the benchmark configurations). Persistent, one CTA per SM.
//
// prefill_kernel: one CTA owns two consecutive 128-row query tiles of one (batch, q head) and
// walks the 64-key KV tiles that the skip range leaves (fully masked tiles are never loaded or
// multiplied). 352 threads:
//   warps 0-3   softmax for query tile 0 (one thread per score row)
//   warps 4-7   softmax for query tile 1
//   warp  8     TMA producer: Q tiles once, then pairs of K/V tiles into a ring, in the order
//               the MMA warps consume them: {K(lo), K(lo+1)}, {V(lo), K(lo+2)}, {V(lo+1), ...
//   warp  9/10  MMA issuers (one thread each, one per query tile): S_t[buf] = Q_t K^T,
//               O_t += P_t V
//
// Tensor memory (512 columns x 128 lanes of 32 bit):
//   tile t, buffer b: S at column t*128 + b*64 (64 fp32 columns); P (bf16, two per column)
//   overwrites the first 32 columns of its S buffer.   O_t at column 256 + t*128 (D columns).
//
// S is double-buffered per query tile: QK^T of KV tile j+2 is issued right after PV of tile j,
// so the tensor pipe computes the next scores while the softmax warps work on the current
// ones; the only dependency left between the two sides is "PV(j) needs P(j)". The softmax warps
// rescale O_t in place when the running max moves by more than 2^8 (rare); "S(k+1) is ready"
// tells them that PV(k-1) is complete.
//
// Shared-memory tiles use the 128-byte swizzle that TMA writes and the MMA descriptors read:
// a [rows][D] bf16 tile is stored as D/64 blocks of [rows][64] (128-byte rows).
// No cluster launch and no multicast: every CTA fetches its own tiles; L2 provides the reuse
// between the CTAs of one kv head.
#include "lf_common.cuh"
#include "lf_skip_range.h"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

#include <atomic>
#include <mutex>
#include <type_traits>

namespace lf {

constexpr int kTileQ = LF_PREFILL_TILE_Q;
constexpr int kTileK = LF_PREFILL_TILE_K;
static_assert(kTileQ == 128 && kTileK == 64, "the kernel is written for 128 x 64 tiles");
constexpr int kPrefillThreads = 11 * 32;  // 8 softmax warps, 1 producer warp, 2 MMA-issuer warps
constexpr int kMaxStages = 16;
constexpr uint32_t kStageBytesTotal = 8 * 2048;
// K/V ring depth in stages of two 64-key tiles: 4 x 32 KB at D=128, 8 x 16 KB at D=64 (which
// also keeps the CTA above half of the shared memory, so two CTAs never compete for the 512
// tensor-memory columns).
template <int D>
struct StagesFor {
  static constexpr int value = D == 64 ? 8 : 4;
};
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // log2 domain
// tanh(x) by odd polynomial: x*(1 - x^2/3) up to |x| <= 0.125 (abs. error < 4.1e-6), degree 7
// up to |x| <= 0.4 (abs. error < 6e-6); MUFU tanh beyond.
constexpr float kTanhPoly1Limit = 0.125f;
constexpr float kTanhPoly3Limit = 0.4f;

constexpr int kModeNone = 0;     // logit2 = raw * c2
constexpr int kModeSoftcap = 1;  // logit2 = tanh(raw * a) * c2
constexpr int kModeGeneric = 2;  // logit2 = mods(raw * a) * c2
// Softcap whose output range is small enough (|c2| <= kBoundedMaxC2) that exp2(logit2) can be
// taken against the fixed reference 0 instead of a running row max: every P lies in
// [2^-80, 2^80], row sums and O stay far inside the fp32 range, and bf16 keeps the same relative
// precision at any magnitude. Without a running max the blocks of a row are independent, there
// is no O rescale, and a row can be split between two threads with no exchange but the final
// row sum.
constexpr int kModeBounded = 3;
constexpr float kBoundedMaxC2 = 80.f;

// Division by a divisor fixed at launch time: q = (mulhi(n, mul) + n) >> shift (Granlund &
// Montgomery's round-up method; exact for every 0 <= n < 2^31). The item decode of the
// persistent kernels runs on one warp that gets few issue slots; real divisions (a few dozen
// dependent instructions each) made it take thousands of clocks.
struct FastDiv {
  uint32_t mul, shift, d;
  static FastDiv make(int32_t divisor) {
    FastDiv f;
    f.d = static_cast<uint32_t>(divisor);
    f.shift = 0;
    while ((1u << f.shift) < f.d) ++f.shift;
    f.mul = static_cast<uint32_t>(((static_cast<uint64_t>(1) << 32) *
                                   ((static_cast<uint64_t>(1) << f.shift) - f.d)) / f.d + 1);
    return f;
  }
  __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
    const uint32_t hi = __umulhi(n, mul);
#else
    const uint32_t hi = static_cast<uint32_t>((static_cast<uint64_t>(n) * mul) >> 32);
#endif
    return static_cast<uint32_t>((static_cast<uint64_t>(hi) + n) >> shift);
  }
};

struct PrefillParams {
  __nv_bfloat16* out;
  int64_t o_stride[3];
  int32_t Sq, Skv, Hq, group;
  int32_t mask_kind, window, causal_offset;
  int32_t n_qtiles;  // ceil(Sq / 128)
  float a;           // multiplies the raw dot product before the score function
  float c2;          // multiplies the score-function output; includes log2(e); > 0
  float qc[4];       // bounded mode: tanh polynomial in raw^2, scaled to give logit2 / raw
  float ylim[2];     // bounded mode: validity limits of the two polynomials, on raw^2
  ModChain mods;
  const __nv_bfloat16* bias;  // additive score bias [B, Hq, Sq, Skv] (generic mode only) or null
  int64_t bias_stride[3];
  int32_t bias_pos;           // the bias is added after this many ops of `mods`
  int32_t* status;
  int32_t* dbg_ranges;
  // Persistent (bounded-mode) kernel only: the work queue.
  int32_t single;        // running-max kernel: one query tile per CTA instead of a pair
  int32_t n_pairs;       // query-tile pairs per head
  int32_t n_deferred;    // persistent kernels: lightest pairs of a head kept for the queue's end
  int32_t main_items;    // (n_pairs - n_deferred) * Hq * B: items ahead of the deferred ones
  FastDiv div_main, div_deferred, div_hq, div_group;  // divisors of the item decode
  int32_t n_items;       // n_pairs * Hq * B
  unsigned int* ticket;  // device counter, zero at launch
  int32_t sm_margin;     // SMs left without a CTA
  // Paged K and / or V (prefill_kernel only): pools [n_pages, page_size, Hkv, D] read through a
  // block table; bit 0 of `paged`: K, bit 1: V.
  int32_t paged;
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  const int32_t* k_table;
  const int32_t* v_table;
  int64_t kp_stride[3], vp_stride[3];  // (page, slot, kv head)
  int64_t bt_stride;
  int32_t page_size, page_shift, n_pages;
  int32_t pe_steps;  // PE variant: 16-column steps of the second score product (D_pe / 16, rounded up)
};

// Barrier block at the start of shared memory.
struct __align__(8) PrefillBarriers {
  uint64_t q_full[2];
  uint64_t kv_full[kMaxStages];
  uint64_t kv_empty[kMaxStages];
  uint64_t s_full[2][2];   // [tile][buffer]  MMA -> softmax
  uint64_t p_full[2][2];   // [tile][buffer]  softmax -> MMA
  uint64_t pv_done[2];     // [tile] second-to-last PV done (running-max modes)
  uint64_t o_final[2];     // [tile] last PV done
  uint32_t tmem_base;
  uint32_t pad;
};

__device__ __forceinline__ void report_timeout(int32_t* status, int where) {
  if (status) atomicCAS(status, LF_DEV_OK, LF_DEV_TIMEOUT | (where << 8));
}

// `PE`: scores are the sum of two products, Q K^T + Q_pe K_pe^T (the two-matmul form of the
// reference's MLA test, tests/test_attention.py:126-151: a "nope" part of width D and a rotary
// part of width D_pe <= 64). The second pair of operands rides along as one more 64-column
// swizzle block behind the D/64 blocks of every Q and K tile - TMA zero-fills the columns past
// D_pe - and the QK^T loop issues its k-steps after the others into the same accumulator. K tiles
// are then larger than V tiles; a ring slot has the size of a K tile.
template <int D, bool PE>
struct PrefillStages {
  static constexpr int value = PE ? (D == 64 ? 4 : 2) : StagesFor<D>::value;
};

template <int D, int MODE, bool PE>
__global__ void __launch_bounds__(kPrefillThreads, 1)
    prefill_kernel(const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v,
                   const __grid_constant__ CUtensorMap tmap_qpe,
                   const __grid_constant__ CUtensorMap tmap_kpe, const PrefillParams p) {
  constexpr int kStages = PrefillStages<D, PE>::value;
  constexpr int kBlocksD = D / 64;                    // 64-column swizzle blocks per tile row
  constexpr int kBlocksQK = kBlocksD + (PE ? 1 : 0);  // ... of a Q or K tile
  constexpr uint32_t kQBlockBytes = kTileQ * 128;     // one [128][64] bf16 block of Q
  constexpr uint32_t kQTileBytes = kQBlockBytes * kBlocksQK;
  constexpr uint32_t kKVBlockBytes = kTileK * 128;    // one [64][64] bf16 block of K or V
  constexpr uint32_t kVTileBytes = kKVBlockBytes * kBlocksD;
  constexpr uint32_t kKTileBytes = kKVBlockBytes * kBlocksQK;
  constexpr uint32_t kKVTileBytes = kKTileBytes;      // size of a ring slot (two per stage)
  constexpr uint32_t kIdescQK = make_idesc_bf16(128, kTileK, 0);
  constexpr uint32_t kIdescPV = make_idesc_bf16(128, D, 1);
  constexpr uint32_t kColO = 256;
  constexpr int kSoftmaxWarps = 8;
  constexpr int kProducerWarp = kSoftmaxWarps;
  constexpr int kMmaWarp0 = kSoftmaxWarps + 1;

  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
  PrefillBarriers* bars = reinterpret_cast<PrefillBarriers*>(smem);
  unsigned char* sStage = smem + 1024;  // 8 x 2 KB: output staging of the softmax warps
  unsigned char* sQ = sStage + kStageBytesTotal;
  unsigned char* sKV = sQ + 2 * kQTileBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Heaviest query tiles first (causal work grows with the row index).
  const int pair = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = h / p.group;
  // (`single`: one query tile per CTA; the second tile slot stays empty. Chosen by the host for
  // problems whose pairs would not fill the SMs: twice the CTAs, each with the tensor pipe and
  // the issue slots of an SM to itself, halve the time of a launch that is a single wave.)
  const int iq0 = p.single ? pair : pair * 2;

  int lo_t[2], hi_t[2];
  skip_range(p.mask_kind, p.window, p.causal_offset, p.Sq, p.Skv, kTileQ, kTileK, iq0, &lo_t[0],
             &hi_t[0]);
  skip_range(p.mask_kind, p.window, p.causal_offset, p.Sq, p.Skv, kTileQ, kTileK, iq0 + 1,
             &lo_t[1], &hi_t[1]);
  const bool tile_valid[2] = {iq0 * kTileQ < p.Sq, !p.single && (iq0 + 1) * kTileQ < p.Sq};
  const bool has_work[2] = {tile_valid[0] && hi_t[0] > lo_t[0], tile_valid[1] && hi_t[1] > lo_t[1]};
  int lo = 0, hi = 0;
  if (has_work[0] && has_work[1]) {
    lo = min(lo_t[0], lo_t[1]);
    hi = max(hi_t[0], hi_t[1]);
  } else if (has_work[0]) {
    lo = lo_t[0];
    hi = hi_t[0];
  } else if (has_work[1]) {
    lo = lo_t[1];
    hi = hi_t[1];
  }

  // ---------------- setup ----------------
  if (warp == kMmaWarp0 && lane == 0) {
    mbar_init(&bars->q_full[0], 1);
    mbar_init(&bars->q_full[1], 1);
    for (int s = 0; s < kStages; ++s) {
      // (paged operands: one arrival for the TMA part, one for the warp's own copies)
      mbar_init(&bars->kv_full[s], p.paged ? 2 : 1);
      mbar_init(&bars->kv_empty[s], 2);
    }
    for (int t = 0; t < 2; ++t) {
      for (int bf = 0; bf < 2; ++bf) {
        mbar_init(&bars->s_full[t][bf], 1);
        mbar_init(&bars->p_full[t][bf], 128);
      }
      mbar_init(&bars->pv_done[t], 1);
      mbar_init(&bars->o_final[t], 1);
    }
    mbar_fence_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == kProducerWarp && p.paged) {
    // ---------------- producer with a paged K and / or V ----------------
    // The two-level load of the reference (loopfuse/codegen.py:738-872: read tile_K table
    // entries, then gather the rows) fused into the tile load: a dense operand still arrives by
    // TMA; a paged one is copied by the whole warp, row by row, with 16-byte cp.async straight
    // from the pool into the 128-byte-swizzled tile layout the MMA descriptors read (16-byte
    // piece c of row r of a 64-column block sits at piece c ^ (r & 7)). Rows past Skv are
    // zero-filled, like TMA does. Copies of up to kLag stages are in flight; a stage is
    // published (second arrival on its full barrier) when its copies have landed and a proxy
    // fence has made them visible to the tensor pipe.
    constexpr int kLag = 2;
    constexpr int kChunks = D / 8;            // 16-byte pieces per row
    constexpr int kRowsPerPass = 32 / kChunks;  // rows one pass of the warp covers
    const bool elected = elect_one_sync();
    if (elected) {
      for (int t = 0; t < 2; ++t) {
        if (!has_work[t]) continue;
        mbar_arrive_expect_tx(&bars->q_full[t], kQTileBytes);
#pragma unroll
        for (int kb = 0; kb < kBlocksD; ++kb)
          tma_load_4d(sQ + t * kQTileBytes + kb * kQBlockBytes, &tmap_q, &bars->q_full[t],
                      kb * 64, (iq0 + t) * kTileQ, h, b);
      }
    }
    __syncwarp();
    int n = 0;
    int published = 0;  // stages whose copies have been published
    bool ok = true;
    auto page_of = [&](int t) { return p.page_shift >= 0 ? (t >> p.page_shift) : (t / p.page_size); };
    // Copy the 64 rows of KV tile j of a paged operand into `dst`.
    auto copy_tile = [&](bool is_v, int j, unsigned char* dst) {
      const __nv_bfloat16* pool = is_v ? p.v_pool : p.k_pool;
      const int32_t* table = (is_v ? p.v_table : p.k_table) + static_cast<int64_t>(b) * p.bt_stride;
      const int64_t* st = is_v ? p.vp_stride : p.kp_stride;
      // Lane l looks up the pages of rows l and l + 32; the others get them by shuffle.
      int64_t row_off[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int t = j * kTileK + half * 32 + lane;
        row_off[half] = -1;
        if (t < p.Skv) {
          const int pg_idx = page_of(t);
          int32_t pg = table[pg_idx];
          if (pg < 0 || pg >= p.n_pages) {
            if (p.status) atomicExch(p.status, LF_DEV_BAD_PAGE);
            pg = 0;
          }
          row_off[half] = pg * st[0] + (t - pg_idx * p.page_size) * st[1] + hkv * st[2];
        }
      }
      const int c = lane % kChunks;
      const uint32_t dst_u32 = smem_u32(dst) + (c / 8) * kKVBlockBytes;
#pragma unroll
      for (int pass = 0; pass < kTileK / kRowsPerPass; ++pass) {
        const int r = pass * kRowsPerPass + lane / kChunks;
        const int64_t off_lo = __shfl_sync(0xffffffffu, row_off[0], r & 31);
        const int64_t off_hi = __shfl_sync(0xffffffffu, row_off[1], r & 31);
        const int64_t off = r < 32 ? off_lo : off_hi;
        const uint32_t d = dst_u32 + r * 128 + (((c & 7) ^ (r & 7)) << 4);
        const __nv_bfloat16* src = pool + (off >= 0 ? off : 0) + c * 8;
        const uint32_t nbytes = off >= 0 ? 16u : 0u;  // 0: the 16 bytes are zero-filled
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src),
                     "r"(nbytes)
                     : "memory");
      }
    };
    auto publish_up_to = [&](int upto) {  // publish stages [published, upto)
      if (published < upto) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0)
          for (int i = published; i < upto; ++i) mbar_arrive(&bars->kv_full[i % kStages]);
        published = upto;
      }
    };
    // ja: tile of `first_is_v ? V : K`; jb >= 0: a K tile in the second half of the stage.
    auto load_pair = [&](bool first_is_v, int ja, int jb) {
      if (!ok) return;
      const int stage = n % kStages;
      const uint32_t parity = ((n / kStages) & 1) ^ 1;
      if (!mbar_wait(&bars->kv_empty[stage], parity)) {
        report_timeout(p.status, 1);
        ok = false;
        return;
      }
      unsigned char* dst = sKV + stage * (2 * kKVTileBytes);
      const bool a_paged = (p.paged >> (first_is_v ? 1 : 0)) & 1;
      const bool b_paged = jb >= 0 && (p.paged & 1);
      if (elected) {
        const uint32_t tx = (a_paged ? 0u : kKVTileBytes) + ((jb >= 0 && !b_paged) ? kKVTileBytes : 0u);
        if (tx) mbar_arrive_expect_tx(&bars->kv_full[stage], tx);
        else mbar_arrive(&bars->kv_full[stage]);
        if (!a_paged) {
#pragma unroll
          for (int kb = 0; kb < kBlocksD; ++kb)
            tma_load_4d(dst + kb * kKVBlockBytes, first_is_v ? &tmap_v : &tmap_k,
                        &bars->kv_full[stage], kb * 64, ja * kTileK, hkv, b);
        }
        if (jb >= 0 && !b_paged) {
#pragma unroll
          for (int kb = 0; kb < kBlocksD; ++kb)
            tma_load_4d(dst + kKVTileBytes + kb * kKVBlockBytes, &tmap_k, &bars->kv_full[stage],
                        kb * 64, jb * kTileK, hkv, b);
        }
      }
      __syncwarp();
      if (a_paged) copy_tile(first_is_v, ja, dst);
      if (b_paged) copy_tile(false, jb, dst + kKVTileBytes);
      cp_async_commit();  // one group per stage, empty or not
      ++n;
      cp_async_wait<kLag>();  // the copies of every stage but the last kLag have landed
      publish_up_to(n - kLag);
    };
    if (hi > lo) {
      load_pair(false, lo, lo + 1 < hi ? lo + 1 : -1);
      for (int j = lo; j < hi; ++j) load_pair(true, j, j + 2 < hi ? j + 2 : -1);
    }
    cp_async_wait<0>();
    publish_up_to(n);
  } else if (warp == kProducerWarp) {
    // ---------------- TMA producer ----------------
    // The whole warp runs the loop and waits; the elected lane issues the copies (a warp that
    // has diverged into a single-lane branch gets few issue slots next to the softmax warps).
    {
      const bool elected = elect_one_sync();
      for (int t = 0; t < 2; ++t) {
        if (!has_work[t]) continue;
        if (elected) {
          mbar_arrive_expect_tx(&bars->q_full[t], kQTileBytes);
#pragma unroll
          for (int kb = 0; kb < kBlocksD; ++kb)
            tma_load_4d(sQ + t * kQTileBytes + kb * kQBlockBytes, &tmap_q, &bars->q_full[t],
                        kb * 64, (iq0 + t) * kTileQ, h, b);
          if constexpr (PE)
            tma_load_4d(sQ + t * kQTileBytes + kBlocksD * kQBlockBytes, &tmap_qpe,
                        &bars->q_full[t], 0, (iq0 + t) * kTileQ, h, b);
        }
        __syncwarp();
      }
      int n = 0;
      bool ok = true;
      // A ring stage holds two 64-key tiles that the MMA warps need at the same time:
      // {K(lo), K(lo+1)} first, then {V(j), K(j+2)} for every j; one full / one empty barrier
      // per stage. `jb < 0` means the second half is not loaded (past the end of the range).
      auto load_pair = [&](const CUtensorMap* tma, int ja, int jb) {
        if (!ok) return;
        const int stage = n % kStages;
        const uint32_t parity = ((n / kStages) & 1) ^ 1;
        ++n;
        if (!mbar_wait(&bars->kv_empty[stage], parity)) {
          report_timeout(p.status, 1);
          ok = false;
          return;
        }
        if (elected) {
          const bool a_is_k = tma == &tmap_k;
          mbar_arrive_expect_tx(&bars->kv_full[stage], (a_is_k ? kKTileBytes : kVTileBytes) +
                                                           (jb >= 0 ? kKTileBytes : 0u));
          unsigned char* dst = sKV + stage * (2 * kKVTileBytes);
#pragma unroll
          for (int kb = 0; kb < kBlocksD; ++kb)
            tma_load_4d(dst + kb * kKVBlockBytes, tma, &bars->kv_full[stage], kb * 64,
                        ja * kTileK, hkv, b);
          if (PE && a_is_k)
            tma_load_4d(dst + kBlocksD * kKVBlockBytes, &tmap_kpe, &bars->kv_full[stage], 0,
                        ja * kTileK, hkv, b);
          if (jb >= 0) {
#pragma unroll
            for (int kb = 0; kb < kBlocksD; ++kb)
              tma_load_4d(dst + kKVTileBytes + kb * kKVBlockBytes, &tmap_k,
                          &bars->kv_full[stage], kb * 64, jb * kTileK, hkv, b);
            if constexpr (PE)
              tma_load_4d(dst + kKVTileBytes + kBlocksD * kKVBlockBytes, &tmap_kpe,
                          &bars->kv_full[stage], 0, jb * kTileK, hkv, b);
          }
        }
        __syncwarp();
      };
      if (hi > lo) {
        load_pair(&tmap_k, lo, lo + 1 < hi ? lo + 1 : -1);
        for (int j = lo; j < hi; ++j) load_pair(&tmap_v, j, j + 2 < hi ? j + 2 : -1);
      }
    }
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // ---------------- MMA issuers: one warp per query tile ----------
    // Two issuing threads halve the per-instruction issue overhead; the tensor pipe serialises
    // the two independent streams. Both walk the same K/V ring and both release every stage
    // (kv_empty counts two arrivals), whether or not their tile used it.
    // The whole warp runs the loop (every lane waits on the barriers); the elected lane alone
    // issues MMAs and commits.
    if (hi > lo) {
      const int t = warp - kMmaWarp0;
      const bool elected = elect_one_sync();
      bool ok = true;
      if (has_work[t] && !mbar_wait(&bars->q_full[t], 0)) {
        report_timeout(p.status, 2);
        ok = false;
      }
      // Descriptors are built once; per MMA only the start-address field moves (in 16-byte
      // units, no carry out of the 14-bit field since shared memory ends below 256 KB).
      constexpr uint32_t kStageUnits = (2 * kKVTileBytes) >> 4;  // a stage is a pair of tiles
      constexpr uint32_t kHalfUnits = kKVTileBytes >> 4;
      const uint64_t qdesc = make_smem_desc_sw128(smem_u32(sQ) + t * kQTileBytes, 16, 1024);
      const uint64_t kdesc0 = make_smem_desc_sw128(smem_u32(sKV), 16, 1024);
      const uint64_t vdesc0 = make_smem_desc_sw128(smem_u32(sKV), kKVBlockBytes, 1024);
      const uint32_t s_col = tmem_base + t * 128;
      const uint32_t o_col = tmem_base + kColO + t * 128;
      int n = 0;  // ring position, walks the same sequence as the producer

      auto active = [&](int j) { return has_work[t] && j >= lo_t[t] && j < hi_t[t]; };
      auto wait_stage = [&](int where) -> int {  // next ring stage, waited full; -1 on time-out
        const int stage = n % kStages;
        const uint32_t parity = (n / kStages) & 1;
        ++n;
        if (!mbar_wait(&bars->kv_full[stage], parity)) {
          report_timeout(p.status, where);
          ok = false;
          return -1;
        }
        return stage;
      };
      // `half` selects the first or second tile of the stage.
      auto issue_qk = [&](int stage, int half, int j) {
        const int buf = (j - lo_t[t]) & 1;
        const uint64_t kd = kdesc0 + static_cast<uint64_t>(stage * kStageUnits + half * kHalfUnits);
        const uint32_t d = s_col + buf * 64;
        if (elected) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            mma_ss(d, qdesc + static_cast<uint64_t>((ks / 4) * (kQBlockBytes >> 4) + (ks % 4) * 2),
                   kd + static_cast<uint64_t>((ks / 4) * (kKVBlockBytes >> 4) + (ks % 4) * 2),
                   kIdescQK, ks > 0 ? 1u : 0u);
          }
          if constexpr (PE) {  // + Q_pe K_pe^T: the extra block of both tiles, same accumulator
            for (int ks = 0; ks < p.pe_steps; ++ks)
              mma_ss(d, qdesc + static_cast<uint64_t>(kBlocksD * (kQBlockBytes >> 4) + ks * 2),
                     kd + static_cast<uint64_t>(kBlocksD * (kKVBlockBytes >> 4) + ks * 2),
                     kIdescQK, 1u);
          }
          tc_commit(&bars->s_full[t][buf]);
        }
        __syncwarp();
      };
      auto issue_pv = [&](int stage, int kt) {
        const uint64_t vd = vdesc0 + static_cast<uint64_t>(stage * kStageUnits);
        const uint32_t a = s_col + (kt & 1) * 64;
        if (elected) {
#pragma unroll
          for (int ks = 0; ks < kTileK / 16; ++ks) {
            mma_ts(o_col, a + ks * 8, vd + static_cast<uint64_t>(ks * (2048 >> 4)), kIdescPV,
                   (kt > 0 || ks > 0) ? 1u : 0u);
          }
        }
        __syncwarp();
      };

      // Prologue: scores of the first two KV tiles (one stage).
      if (ok) {
        const int stage = wait_stage(3);
        if (stage >= 0) {
          tc_fence_after();
          if (active(lo)) issue_qk(stage, 0, lo);
          if (lo + 1 < hi && active(lo + 1)) issue_qk(stage, 1, lo + 1);
          if (elected) tc_commit(&bars->kv_empty[stage]);
          __syncwarp();
        }
      }
      const int nblk_t = has_work[t] ? hi_t[t] - lo_t[t] : 0;
      for (int j = lo; j < hi && ok; ++j) {
        const int st = wait_stage(4);  // {V(j), K(j+2)}
        if (st < 0) break;
        tc_fence_after();
        if (active(j)) {
          const int kt = j - lo_t[t];
          if (!mbar_wait(&bars->p_full[t][kt & 1], (kt >> 1) & 1)) {
            report_timeout(p.status, 6 + t);
            ok = false;
            break;
          }
          tc_fence_after();
          issue_pv(st, kt);
          // Completion points the softmax warps may wait on: the second-to-last PV (for a
          // rescale in the last block) and the last PV (for the epilogue).
          if (elected) {
            if (kt == nblk_t - 2) tc_commit(&bars->pv_done[t]);
            if (kt == nblk_t - 1) tc_commit(&bars->o_final[t]);
          }
        }
        if (j + 2 < hi && active(j + 2)) issue_qk(st, 1, j + 2);
        if (elected) tc_commit(&bars->kv_empty[st]);
        __syncwarp();
      }
    }
  } else {
    // ---------------- softmax warps ----------------
    const int t = warp >> 2;                 // query tile of this warp group
    const int row = (warp & 3) * 32 + lane;  // row inside the tile == tensor-memory lane
    const int grow = (iq0 + t) * kTileQ + row;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_base = tmem_base + lane_addr + t * 128;
    const uint32_t o_addr = tmem_base + lane_addr + kColO + t * 128;

    if (p.dbg_ranges && tile_valid[t] && row == 0) {
      const int64_t idx = ((static_cast<int64_t>(b) * p.Hq + h) * p.n_qtiles + (iq0 + t)) * 2;
      p.dbg_ranges[idx] = lo_t[t];
      p.dbg_ranges[idx + 1] = hi_t[t];
    }

    if (has_work[t]) {
      // Visible column interval of this row: [c_lo, c_hi].
      int c_hi = p.Skv - 1;
      int c_lo = 0;
      if (p.mask_kind != LF_MASK_NONE) c_hi = min(c_hi, grow + p.causal_offset);
      if (p.mask_kind == LF_MASK_CAUSAL_WINDOW)
        c_lo = max(0, grow + p.causal_offset - (p.window - 1));

      float m_used = -INFINITY;  // max the stored P and O are scaled by (log2 domain)
      float l_run = 0.f;
      bool ok = true;
      const int nblk = hi_t[t] - lo_t[t];
      for (int k = 0; k < nblk; ++k) {
        const int c0 = (lo_t[t] + k) * kTileK;
        const int buf = k & 1;
        const uint32_t s_addr = s_base + buf * 64;
        if (!mbar_wait(&bars->s_full[t][buf], (k >> 1) & 1)) {
          report_timeout(p.status, 8 + t);
          ok = false;
          break;
        }
        tc_fence_after();
        // Raw scores of this row: 64 fp32 values.
        uint32_t sr[2][32];
        tmem_ld_32x32b_x32(s_addr, sr[0]);
        tmem_ld_32x32b_x32(s_addr + 32, sr[1]);
        tmem_wait_ld();

        const int rel_lo = c_lo - c0;  // visible columns of this row inside the tile:
        const int rel_hi = c_hi - c0;  // [rel_lo, rel_hi]
        const bool masked = rel_lo > 0 || rel_hi < kTileK - 1;

        if constexpr (MODE == kModeGeneric) {
          // The chain is interpreted op by op over the row's 64 scores in registers: one
          // (warp-uniform) dispatch per op and block, not one per score - the reference compiles
          // a kernel per chain (loopfuse/codegen.py:454-998), an interpreter has to keep its
          // dispatch out of the element loop.
          auto each = [&](auto f) {
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                sr[c][i] = __float_as_uint(f(__uint_as_float(sr[c][i])));
          };
          auto run_mods = [&](int m_lo, int m_hi) {
#pragma unroll 1
            for (int m = m_lo; m < m_hi; ++m) {
              const float a = p.mods.arg[m];
              switch (p.mods.op[m]) {
                case LF_MOD_MUL: each([&](float x) { return x * a; }); break;
                case LF_MOD_ADD: each([&](float x) { return x + a; }); break;
                case LF_MOD_TANH: each([&](float x) { return tanhf(x); }); break;
                case LF_MOD_EXP: each([&](float x) { return __expf(x); }); break;
                case LF_MOD_EXP2: each([&](float x) { return exp2f(x); }); break;
                case LF_MOD_SIN: each([&](float x) { return sinf(x); }); break;
                case LF_MOD_COS: each([&](float x) { return cosf(x); }); break;
                case LF_MOD_RELU: each([&](float x) { return fmaxf(x, 0.f); }); break;
                case LF_MOD_SQUARE: each([&](float x) { return x * x; }); break;
                case LF_MOD_DIV: each([&](float x) { return x / a; }); break;
                default: break;
              }
            }
          };
          each([&](float x) { return x * p.a; });
          if (p.bias == nullptr) {
            run_mods(0, p.mods.n);
          } else {
            run_mods(0, p.bias_pos);
            // This row's 64 bias values of the block: 128 contiguous bytes, eight 16-byte loads
            // (rows past Sq read the last row, columns past Skv are not read: both are masked
            // or clipped later).
            const __nv_bfloat16* brow = p.bias + b * p.bias_stride[0] + h * p.bias_stride[1] +
                                        static_cast<int64_t>(min(grow, p.Sq - 1)) * p.bias_stride[2] +
                                        c0;
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i8 = 0; i8 < 4; ++i8) {
                const int cc = c * 32 + i8 * 8;
                uint32_t w[4] = {0u, 0u, 0u, 0u};
                if (c0 + cc + 8 <= p.Skv &&
                    LF_BOUNDS(c0 + cc >= 0 && b < static_cast<int>(gridDim.z) && h < p.Hq,
                              p.status, 60)) {
                  const uint4 v4 = ldg_stream_16(brow + cc);
                  w[0] = v4.x; w[1] = v4.y; w[2] = v4.z; w[3] = v4.w;
                } else {
#pragma unroll
                  for (int e = 0; e < 8; ++e)
                    if (c0 + cc + e < p.Skv)
                      w[e >> 1] |= static_cast<uint32_t>(__bfloat16_as_ushort(brow[cc + e]))
                                   << ((e & 1) * 16);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float bv = __uint_as_float((e & 1) ? (w[e >> 1] & 0xffff0000u)
                                                           : (w[e >> 1] << 16));
                  sr[c][i8 * 8 + e] = __float_as_uint(__uint_as_float(sr[c][i8 * 8 + e]) + bv);
                }
              }
            run_mods(p.bias_pos, p.mods.n);
          }
        }

        // Pass 1: row max (and min, for the softcap range check), independent chains.
        float mxa[4], mna[4];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          mxa[2 * c] = mxa[2 * c + 1] = -INFINITY;
          mna[2 * c] = mna[2 * c + 1] = INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float v0 = __uint_as_float(sr[c][i]), v1 = __uint_as_float(sr[c][i + 1]);
            const float v2 = __uint_as_float(sr[c][i + 2]), v3 = __uint_as_float(sr[c][i + 3]);
            mxa[2 * c] = max3(mxa[2 * c], v0, v1);
            mxa[2 * c + 1] = max3(mxa[2 * c + 1], v2, v3);
            if constexpr (MODE == kModeSoftcap) {
              mna[2 * c] = min3(mna[2 * c], v0, v1);
              mna[2 * c + 1] = min3(mna[2 * c + 1], v2, v3);
            }
          }
        }
        const float mx_all = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
        float mx_keep = mx_all;
        if (masked) {  // max over the visible columns only
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            mxa[c] = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int cc = c * 32 + i;
              const float v = (cc >= rel_lo && cc <= rel_hi) ? __uint_as_float(sr[c][i]) : -INFINITY;
              mxa[c] = fmaxf(mxa[c], v);
            }
          }
          mx_keep = fmaxf(mxa[0], mxa[1]);
        }

        // The score function is monotonic for the plain and softcap modes, so the max of the
        // scores is the score of the max.
        float tmax = mx_keep;
        unsigned flags = 0;  // bit 0: |x| > poly-1 limit, bit 1: |x| > poly-3 limit, bit 2: rescale
        if constexpr (MODE == kModeSoftcap) {
          tmax = (mx_keep == -INFINITY) ? -INFINITY : tanh_approx(mx_keep * p.a);
          // Every |x| of the warp's rows decides (masked columns included: their raw scores
          // are ordinary finite numbers).
          const float mn_all = fminf(fminf(mna[0], mna[1]), fminf(mna[2], mna[3]));
          const float bound = fabsf(p.a) * fmaxf(fabsf(mx_all), fabsf(mn_all));
          flags = (bound > kTanhPoly1Limit ? 1u : 0u) | (bound > kTanhPoly3Limit ? 2u : 0u);
        }
        const float m_new = fmaxf(m_used, tmax * p.c2);

        // Lazy rescale: move the reference max only when it grew by more than 2^8.
        float alpha = 1.f;
        if (m_new > -INFINITY && (m_used == -INFINITY || m_new - m_used > kRescaleThreshold)) {
          flags |= 4u;
          alpha = ex2_approx(m_used - m_new);  // 0 when m_used is -inf
          m_used = m_new;
        }
        flags = __reduce_or_sync(0xffffffffu, flags);  // one vote for all warp-level decisions
        // 0: x*(1 - x^2/3), 1: degree-7 polynomial, 2: MUFU tanh
        const int tanh_path = (flags & 2u) ? 2 : ((flags & 1u) ? 1 : 0);
        if (k > 0 && (flags & 4u)) {
          // O_t must hold every PV up to k-1 and none may be in flight. QK(k+1) is issued after
          // PV(k-1), so "S(k+1) is ready" implies it; in the last block there is no S(k+1) and
          // the MMA warp commits pv_done after the second-to-last PV instead.
          const bool last = k + 1 == nblk;
          uint64_t* bar = last ? &bars->pv_done[t] : &bars->s_full[t][(k + 1) & 1];
          if (!mbar_wait(bar, last ? 0u : (((k + 1) >> 1) & 1))) {
            report_timeout(p.status, 12 + t);
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t orr[32];
            tmem_ld_32x32b_x32(o_addr + c * 32, orr);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
            tmem_st_32x32b_x32(o_addr + c * 32, orr);
          }
        }
        const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;

        // Pass 2: p = exp2(score * c2 - m). Plain fp32 instructions and every exp2 on MUFU: the
        // loop is bound by instruction issue, and the packed f32x2 forms (fewer instructions,
        // but slower in their pipe) and an FMA-pipe emulation of part of the exp2 both measured
        // slower than this in the fixed-reference kernel, which runs the same arithmetic.
        const float neg_m = -m_safe;
        float ps[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[32];
        auto finish_pair = [&](float z0, float z1, int c, int i, bool apply_mask) {
          if (apply_mask) {
            const int cc = c * 32 + i;
            if (cc < rel_lo || cc > rel_hi) z0 = -INFINITY;
            if (cc + 1 < rel_lo || cc + 1 > rel_hi) z1 = -INFINITY;
          }
          const float p0 = ex2_approx(z0), p1 = ex2_approx(z1);
          ps[(c * 2 + (i >> 1)) & 3] += p0;
          ps[(c * 2 + (i >> 1) + 2) & 3] += p1;
          pk[c * 16 + (i >> 1)] = pack_bf16x2(p0, p1);
        };
        if (MODE == kModeSoftcap && tanh_path < 2) {
          // tanh(x) = x*(1 + y*(-1/3 + y*(2/15 + y*(-17/315)))), y = x^2, x = a*raw; the powers
          // of a are folded into the coefficients so that the polynomial runs on raw^2.
          const float a2 = p.a * p.a;
          const float b1 = -a2 / 3.f;
          const float ac = p.a * p.c2;
          if (tanh_path == 0) {
            auto body = [&](bool apply_mask) {
#pragma unroll
              for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  const float r0 = __uint_as_float(sr[c][i]), r1 = __uint_as_float(sr[c][i + 1]);
                  const float q0 = fmaf(r0 * r0, b1, 1.f), q1 = fmaf(r1 * r1, b1, 1.f);
                  finish_pair(fmaf(r0 * ac, q0, neg_m), fmaf(r1 * ac, q1, neg_m), c, i,
                              apply_mask);
                }
            };
            if (masked) body(true); else body(false);
          } else {
            const float b2 = a2 * a2 * (2.f / 15.f);
            const float b3 = a2 * a2 * a2 * (-17.f / 315.f);
            auto body = [&](bool apply_mask) {
#pragma unroll
              for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  const float r0 = __uint_as_float(sr[c][i]), r1 = __uint_as_float(sr[c][i + 1]);
                  const float y0 = r0 * r0, y1 = r1 * r1;
                  const float q0 = fmaf(fmaf(fmaf(y0, b3, b2), y0, b1), y0, 1.f);
                  const float q1 = fmaf(fmaf(fmaf(y1, b3, b2), y1, b1), y1, 1.f);
                  finish_pair(fmaf(r0 * ac, q0, neg_m), fmaf(r1 * ac, q1, neg_m), c, i,
                              apply_mask);
                }
            };
            if (masked) body(true); else body(false);
          }
        } else if constexpr (MODE == kModeSoftcap) {
          auto body = [&](bool apply_mask) {
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float t0 = tanh_approx(__uint_as_float(sr[c][i]) * p.a);
                const float t1 = tanh_approx(__uint_as_float(sr[c][i + 1]) * p.a);
                finish_pair(fmaf(t0, p.c2, neg_m), fmaf(t1, p.c2, neg_m), c, i, apply_mask);
              }
          };
          if (masked) body(true); else body(false);
        } else {
          auto body = [&](bool apply_mask) {
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i = 0; i < 32; i += 2)
                finish_pair(fmaf(__uint_as_float(sr[c][i]), p.c2, neg_m),
                            fmaf(__uint_as_float(sr[c][i + 1]), p.c2, neg_m), c, i, apply_mask);
          };
          if (masked) body(true); else body(false);
        }
        const float psum = (ps[0] + ps[1]) + (ps[2] + ps[3]);
        l_run = l_run * alpha + psum;
        tmem_st_32x32b_x32(s_addr, pk);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full[t][buf]);
      }

      // Epilogue: O_t / l -> bf16 -> global (one row per thread).
      if (ok) {
        if (!mbar_wait(&bars->o_final[t], 0)) {
          report_timeout(p.status, 10 + t);
          ok = false;
        }
      }
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / l_run;
        // Each warp owns 32 rows. A 32-column chunk (64 bytes per row) goes through a swizzled
        // 2 KB buffer of the warp so that one store instruction writes eight 64-byte row
        // segments instead of thirty-two 16-byte pieces.
        unsigned char* stage = sStage + warp * 2048;
        __nv_bfloat16* obase = p.out + b * p.o_stride[0] + h * p.o_stride[1];
        const int row0 = (iq0 + t) * kTileQ + (warp & 3) * 32;  // first global row of the warp
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld_32x32b_x32(o_addr + c * 32, orr);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 4; ++q) {  // piece q of row r sits at position q ^ ((r >> 1) & 3)
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(orr[8 * q]) * inv,
                              __uint_as_float(orr[8 * q + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(orr[8 * q + 2]) * inv,
                              __uint_as_float(orr[8 * q + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(orr[8 * q + 4]) * inv,
                              __uint_as_float(orr[8 * q + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(orr[8 * q + 6]) * inv,
                              __uint_as_float(orr[8 * q + 7]) * inv);
            *reinterpret_cast<uint4*>(stage + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) = w;
          }
          __syncwarp();
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int r = rr * 8 + (lane >> 2);
            const int q = lane & 3;
            const uint4 w =
                *reinterpret_cast<const uint4*>(stage + r * 64 + ((q ^ ((r >> 1) & 3)) << 4));
            if (row0 + r < p.Sq)
              *reinterpret_cast<uint4*>(obase + static_cast<int64_t>(row0 + r) * p.o_stride[2] +
                                        c * 32 + q * 8) = w;
          }
          __syncwarp();
        }
      }
    } else if (tile_valid[t] && grow < p.Sq) {
      // No visible key at all for this tile: softmax of an all -inf row is NaN in the
      // eager computation, so the rows are written as NaN.
      __nv_bfloat16* orow = p.out + b * p.o_stride[0] + h * p.o_stride[1] +
                            static_cast<int64_t>(grow) * p.o_stride[2];
      const uint4 nan4 = {0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u};
#pragma unroll
      for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = nan4;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace lf

#include "lf_prefill_bounded.cuh"
#include "lf_prefill_wide.cuh"

namespace lf {

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000,
                                                     cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    else
      set_cuda_error(e, "cudaGetDriverEntryPointByVersion(cuTensorMapEncodeTiled)");
  });
  return fn;
}

// Tensor map over a bf16 [B, H, S, D] tensor (innermost stride 1), box = [1, 1, box_rows,
// box_cols]; 128-byte swizzle for 64-column boxes (the K/V/Q loads, out-of-range rows read as
// zero), 64-byte swizzle for 32-column boxes (the output store of the persistent kernels).
static int encode_tile_map(CUtensorMap* map, const void* base, int B, int H, int S, int D,
                           const int64_t* stride /* b, h, s in elements */, int box_rows,
                           int box_cols) {
  auto fn = get_encode_fn();
  if (!fn) return LF_ERR_CUDA;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S),
                        static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(stride[2]) * 2,
                           static_cast<cuuint64_t>(stride[1]) * 2,
                           static_cast<cuuint64_t>(stride[0]) * 2};
  // A dimension of extent 1 may carry any stride; keep it a valid multiple of 16 bytes.
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0 || (strides[i] & 15)) {
      if (dims[i + 1] == 1)
        strides[i] = 16 * ((static_cast<cuuint64_t>(D) * 2 + 15) / 16);
      else
        return LF_ERR_ALIGNMENT;
    }
  cuuint32_t box[4] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return LF_ERR_CUDA;
  }
  return LF_OK;
}

// Encoded tensor maps are kept in a small cache: a map depends only on (address, shape,
// strides, box), and serving loops call with the same buffers again and again. Direct-mapped,
// one mutex; a miss just encodes again, so the cache never changes a result. A CUtensorMap holds
// no reference to the memory it describes: an entry whose buffer was freed is harmless and is
// simply replaced when another key lands on its slot.
struct TileMapKey {
  const void* base;
  int32_t B, H, S, D, box_rows, box_cols;
  int64_t stride[3];
  bool operator==(const TileMapKey& o) const {
    return base == o.base && B == o.B && H == o.H && S == o.S && D == o.D &&
           box_rows == o.box_rows && box_cols == o.box_cols && stride[0] == o.stride[0] &&
           stride[1] == o.stride[1] && stride[2] == o.stride[2];
  }
};
struct TileMapEntry {
  bool valid = false;
  TileMapKey key;
  CUtensorMap map;
};
constexpr int kTileMapCacheSlots = 256;
static std::mutex g_tile_map_mutex;
static TileMapEntry g_tile_map_cache[kTileMapCacheSlots];
static std::atomic<uint64_t> g_tile_map_hits{0}, g_tile_map_misses{0};

static int make_tile_map(CUtensorMap* map, const void* base, int B, int H, int S, int D,
                         const int64_t* stride, int box_rows, int box_cols = 64) {
  TileMapKey key{base, B, H, S, D, box_rows, box_cols, {stride[0], stride[1], stride[2]}};
  uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
  h ^= (static_cast<uint64_t>(S) << 32 | static_cast<uint32_t>(H)) * 0xC2B2AE3D27D4EB4Full;
  h ^= (static_cast<uint64_t>(B) << 40 | static_cast<uint64_t>(box_rows) << 16 |
        static_cast<uint64_t>(box_cols) << 8 | static_cast<uint64_t>(D)) * 0x165667B19E3779F9ull;
  h ^= static_cast<uint64_t>(stride[2]) * 0x27D4EB2F165667C5ull;
  const int slot = static_cast<int>((h >> 32) % kTileMapCacheSlots);
  {
    std::lock_guard<std::mutex> lock(g_tile_map_mutex);
    const TileMapEntry& e = g_tile_map_cache[slot];
    if (e.valid && e.key == key) {
      *map = e.map;
      g_tile_map_hits.fetch_add(1, std::memory_order_relaxed);
      return LF_OK;
    }
  }
  const int rc = encode_tile_map(map, base, B, H, S, D, stride, box_rows, box_cols);
  if (rc != LF_OK) return rc;
  g_tile_map_misses.fetch_add(1, std::memory_order_relaxed);
  std::lock_guard<std::mutex> lock(g_tile_map_mutex);
  TileMapEntry& e = g_tile_map_cache[slot];
  e.key = key;
  e.map = *map;
  e.valid = true;
  return LF_OK;
}

template <int D, int MODE, bool PE = false>
static int launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                          const PrefillParams& p, int B, cudaStream_t st,
                          const CUtensorMap* mqpe = nullptr, const CUtensorMap* mkpe = nullptr) {
  constexpr size_t kQTileBytes = static_cast<size_t>(kTileQ) * (D + (PE ? 64 : 0)) * 2;
  constexpr size_t kKVTileBytes = static_cast<size_t>(kTileK) * (D + (PE ? 64 : 0)) * 2;
  constexpr size_t smem = 1024 /*align slack*/ + 1024 /*barriers*/ + kStageBytesTotal +
                          2 * kQTileBytes +
                          PrefillStages<D, PE>::value * 2 * kKVTileBytes;
  static_assert(smem <= 232448, "shared memory of a CTA");
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel<D, MODE, PE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) {
      set_cuda_error(e, "cudaFuncSetAttribute(prefill_kernel)");
      return LF_ERR_CUDA;
    }
    configured_dev = dev;
  }
  const int pairs = (p.n_qtiles + 1) / 2;
  static thread_local int sm_count = 0;
  if (sm_count == 0) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  PrefillParams pp = p;
  pp.single = (p.n_qtiles > 1 && static_cast<int64_t>(pairs) * p.Hq * B < sm_count) ? 1 : 0;
  dim3 grid(pp.single ? p.n_qtiles : pairs, p.Hq, B);
  // (without a second score product the two extra maps are never read)
  prefill_kernel<D, MODE, PE><<<grid, kPrefillThreads, smem, st>>>(mq, mk, mv, mqpe ? *mqpe : mq,
                                                                   mkpe ? *mkpe : mk, pp);
  return check_launch("prefill_kernel");
}

// Ticket counters of the persistent kernel: a small ring in the library image, so that launching
// allocates nothing. A launch takes the next slot and zeroes it in stream order; launches that
// overlap on the GPU use different slots unless more than kTicketSlots are in flight.
constexpr int kTicketSlots = 256;
static __device__ unsigned int g_prefill_tickets[kTicketSlots];
static std::atomic<unsigned int> g_next_ticket_slot{0};

template <int D, int PACK = 1>
static int launch_prefill_bounded(const CUtensorMap& mq, const CUtensorMap& mk,
                                  const CUtensorMap& mv, const CUtensorMap& mo, PrefillParams p,
                                  int B, cudaStream_t st) {
  constexpr size_t kQTileBytes = static_cast<size_t>(kTileQ) * D * 2;
  constexpr size_t kKVTileBytes = static_cast<size_t>(kTileK) * D * 2;
  constexpr bool kBig = PACK > 1 && D == 128;
  constexpr size_t smem = 1024 /*align slack*/ + 1024 /*barriers*/ +
                          (kBig ? 16 * 4096 : kBoundedStageBytes) + 2 * kQTileBytes +
                          (kBig ? 3 : StagesFor<D>::value) * 2 * kKVTileBytes;
  static_assert(smem <= 232448, "smem");
  static thread_local int configured_dev = -1;
  static thread_local unsigned int* tickets = nullptr;
  static thread_local int sm_count = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(prefill_bounded_kernel<D, PACK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e == cudaSuccess)
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&tickets), g_prefill_tickets);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      set_cuda_error(e, "prefill_bounded_kernel setup");
      return LF_ERR_CUDA;
    }
    configured_dev = dev;
  }
  // Packed layout: the query rows are walked in chunks of 128 / PACK (p.n_qtiles counts those) and an
  // item is a pair of chunks of one kv head, for all of its query heads at once.
  const int heads = PACK > 1 ? p.Hq / p.group : p.Hq;
  if (PACK > 1) p.n_qtiles = (p.Sq + kTileQ / PACK - 1) / (kTileQ / PACK);
  p.n_pairs = (p.n_qtiles + 1) / 2;
  p.n_deferred = (p.mask_kind == LF_MASK_CAUSAL && p.Sq == p.Skv) ? p.n_pairs / 4 : 0;
  p.main_items = static_cast<int32_t>(static_cast<int64_t>(p.n_pairs - p.n_deferred) * heads * B);
  p.div_main = FastDiv::make(p.n_pairs - p.n_deferred);
  p.div_deferred = FastDiv::make(p.n_deferred > 0 ? p.n_deferred : 1);
  p.div_hq = FastDiv::make(heads);
  p.div_group = FastDiv::make(p.group);
  const int64_t n_items = static_cast<int64_t>(p.n_pairs) * heads * B;
  if (n_items > 0x7fffffff - 4096) return LF_ERR_TOO_LARGE;
  p.n_items = static_cast<int32_t>(n_items);
  p.ticket = tickets + g_next_ticket_slot.fetch_add(1) % kTicketSlots;
  cudaError_t e = cudaMemsetAsync(p.ticket, 0, sizeof(unsigned int), st);
  if (e != cudaSuccess) {
    set_cuda_error(e, "cudaMemsetAsync(ticket)");
    return LF_ERR_CUDA;
  }
  const int ctas = sm_count - p.sm_margin > 0 ? sm_count - p.sm_margin : 1;
  const int grid = static_cast<int>(n_items < ctas ? n_items : ctas);
  prefill_bounded_kernel<D, PACK><<<grid, kBoundedThreads, smem, st>>>(mq, mk, mv, mo, p);
  return check_launch("prefill_bounded_kernel");
}

template <int D>
static int launch_prefill_wide(const CUtensorMap& mq, const CUtensorMap& mk,
                               const CUtensorMap& mv, const CUtensorMap& mo, PrefillParams p,
                               int B, cudaStream_t st) {
  constexpr size_t kQTileBytes = static_cast<size_t>(kTileQ) * D * 2;
  constexpr size_t kKVTileBytes = static_cast<size_t>(kWideK) * D * 2;
  constexpr size_t smem = 1024 /*align slack*/ + 1024 /*barriers*/ + kBoundedStageBytes +
                          2 * kQTileBytes + WideRingFor<D>::value * kKVTileBytes;
  static thread_local int configured_dev = -1;
  static thread_local unsigned int* tickets = nullptr;
  static thread_local int sm_count = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(prefill_wide_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e == cudaSuccess)
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&tickets), g_prefill_tickets);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      set_cuda_error(e, "prefill_wide_kernel setup");
      return LF_ERR_CUDA;
    }
    configured_dev = dev;
  }
  p.n_pairs = (p.n_qtiles + 1) / 2;
  p.n_deferred = (p.mask_kind == LF_MASK_CAUSAL && p.Sq == p.Skv) ? p.n_pairs / 4 : 0;
  p.main_items = static_cast<int32_t>(static_cast<int64_t>(p.n_pairs - p.n_deferred) * p.Hq * B);
  p.div_main = FastDiv::make(p.n_pairs - p.n_deferred);
  p.div_deferred = FastDiv::make(p.n_deferred > 0 ? p.n_deferred : 1);
  p.div_hq = FastDiv::make(p.Hq);
  p.div_group = FastDiv::make(p.group);
  const int64_t n_items = static_cast<int64_t>(p.n_pairs) * p.Hq * B;
  if (n_items > 0x7fffffff - 4096) return LF_ERR_TOO_LARGE;
  p.n_items = static_cast<int32_t>(n_items);
  p.ticket = tickets + g_next_ticket_slot.fetch_add(1) % kTicketSlots;
  cudaError_t e = cudaMemsetAsync(p.ticket, 0, sizeof(unsigned int), st);
  if (e != cudaSuccess) {
    set_cuda_error(e, "cudaMemsetAsync(ticket)");
    return LF_ERR_CUDA;
  }
  const int ctas = sm_count - p.sm_margin > 0 ? sm_count - p.sm_margin : 1;
  const int grid = static_cast<int>(n_items < ctas ? n_items : ctas);
  prefill_wide_kernel<D><<<grid, kWideThreads, smem, st>>>(mq, mk, mv, mo, p);
  return check_launch("prefill_wide_kernel");
}

// KV tile of the kernel that serves these arguments. The bounded-softcap mode has two kernels:
// 64-key tiles (two S buffers per query tile, the default: the faster of the two on every
// configuration measured) and 128-key tiles (one S buffer, math-bound N=128 QK^T MMAs), which a
// caller can pin with kv_tile = 128. Every running-max kernel uses 64-key tiles.
static int choose_kv_tile(const LfPrefillArgs* a, int mode) {
  if (a->kv_tile != 0 && a->kv_tile != kTileK && a->kv_tile != kWideK) return LF_ERR_INVALID_ARG;
  if (mode != kModeBounded) return a->kv_tile == kWideK ? LF_ERR_UNSUPPORTED : kTileK;
  return a->kv_tile != 0 ? a->kv_tile : kTileK;
}

// `launch` == nullptr: only resolve the kernel choice and return its KV tile size.
static int prefill_impl(const LfPrefillArgs* a, void* const* launch, int* q_tile = nullptr) {
  if (!a || !a->q || !a->k || !a->v || !a->out) return LF_ERR_INVALID_ARG;
  if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Sq <= 0 || a->Skv <= 0)
    return LF_ERR_INVALID_ARG;
  if (a->Hq % a->Hkv) return LF_ERR_INVALID_ARG;
  if (a->D != 64 && a->D != 128) return LF_ERR_UNSUPPORTED;
  if (a->n_mod < 0 || a->n_mod > LF_MAX_MODS) return LF_ERR_INVALID_ARG;
  if (a->mask_kind < LF_MASK_NONE || a->mask_kind > LF_MASK_CAUSAL_WINDOW)
    return LF_ERR_INVALID_ARG;
  if (a->mask_kind == LF_MASK_CAUSAL_WINDOW && a->window <= 0) return LF_ERR_INVALID_ARG;
  if (a->Hq > 65535 || a->B > 65535) return LF_ERR_TOO_LARGE;
  const void* ptrs[4] = {a->q, a->k, a->v, a->out};
  for (const void* ptr : ptrs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15u) return LF_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if (a->o_stride[i] % 8) return LF_ERR_ALIGNMENT;

  PrefillParams p;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  for (int i = 0; i < 3; ++i) p.o_stride[i] = a->o_stride[i];
  p.Sq = a->Sq;
  p.Skv = a->Skv;
  p.Hq = a->Hq;
  p.group = a->Hq / a->Hkv;
  p.mask_kind = a->mask_kind;
  p.window = a->window;
  p.causal_offset = a->causal_offset;
  p.n_qtiles = (a->Sq + kTileQ - 1) / kTileQ;
  p.status = a->status;
  p.dbg_ranges = a->dbg_ranges;
  for (int i = 0; i < 4; ++i) p.qc[i] = 0.f;
  p.ylim[0] = p.ylim[1] = 0.f;
  p.single = 0;
  p.n_pairs = 0;
  p.n_deferred = 0;
  p.main_items = 0;
  p.div_main = p.div_deferred = p.div_hq = p.div_group = FastDiv::make(1);
  p.n_items = 0;
  p.ticket = nullptr;
  if (a->sm_margin < 0) return LF_ERR_INVALID_ARG;
  p.sm_margin = a->sm_margin;
  // Paged operands: `k` / `v` is then a pool [n_pages, page_size, Hkv, D] with strides (page,
  // slot, kv head), read through its block table.
  p.paged = (a->k_block_table ? 1 : 0) | (a->v_block_table ? 2 : 0);
  p.k_pool = static_cast<const __nv_bfloat16*>(a->k);
  p.v_pool = static_cast<const __nv_bfloat16*>(a->v);
  p.k_table = a->k_block_table;
  p.v_table = a->v_block_table;
  for (int i = 0; i < 3; ++i) {
    p.kp_stride[i] = a->k_stride[i];
    p.vp_stride[i] = a->v_stride[i];
  }
  p.bt_stride = a->bt_stride;
  p.page_size = a->page_size;
  p.page_shift = -1;
  p.n_pages = a->n_pages;
  if (p.paged) {
    if (a->page_size <= 0 || a->n_pages <= 0) return LF_ERR_INVALID_ARG;
    if (a->bt_stride < (a->Skv + a->page_size - 1) / a->page_size) return LF_ERR_INVALID_ARG;
    for (int sh = 0; sh < 31; ++sh)
      if ((1 << sh) == a->page_size) p.page_shift = sh;
    for (int i = 0; i < 3; ++i)
      if (((p.paged & 1) && a->k_stride[i] % 8) || ((p.paged & 2) && a->v_stride[i] % 8))
        return LF_ERR_ALIGNMENT;
  }
  p.mods.n = 0;
  for (int i = 0; i < LF_MAX_MODS; ++i) {
    p.mods.op[i] = 0;
    p.mods.arg[i] = 0.f;
  }
  p.pe_steps = 0;
  const bool has_pe = a->q_pe != nullptr || a->k_pe != nullptr;
  if (has_pe) {
    if (!a->q_pe || !a->k_pe) return LF_ERR_INVALID_ARG;
    if (a->D_pe <= 0 || a->D_pe > 64 || a->D_pe % 8) return LF_ERR_UNSUPPORTED;
    if (p.paged || a->score_bias) return LF_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a->q_pe) | reinterpret_cast<uintptr_t>(a->k_pe)) & 15u)
      return LF_ERR_ALIGNMENT;
    p.pe_steps = (a->D_pe + 15) / 16;
  }
  p.bias = static_cast<const __nv_bfloat16*>(a->score_bias);
  p.bias_pos = a->bias_pos;
  for (int i = 0; i < 3; ++i) p.bias_stride[i] = a->bias_stride[i];
  if (p.bias) {
    if (p.paged) return LF_ERR_UNSUPPORTED;
    if (a->bias_pos < 0 || a->bias_pos > a->n_mod) return LF_ERR_INVALID_ARG;
    if (reinterpret_cast<uintptr_t>(a->score_bias) & 15u) return LF_ERR_ALIGNMENT;
    for (int i = 0; i < 3; ++i)
      if (a->bias_stride[i] % 8) return LF_ERR_ALIGNMENT;
  }

  // Pick the score-function mode. Leading and trailing constant multipliers are folded into
  // `a` (before) and `c2` (after); c2 must stay positive for the max-before-scale shortcut.
  int mode = kModeGeneric;
  if (!p.bias) {  // (a score bias always takes the generic path: the chain is split around it)
    int i = 0;
    float pre = a->scale;
    while (i < a->n_mod && (a->mod_op[i] == LF_MOD_MUL || a->mod_op[i] == LF_MOD_DIV)) {
      pre = a->mod_op[i] == LF_MOD_MUL ? pre * a->mod_arg[i] : pre / a->mod_arg[i];
      ++i;
    }
    if (i == a->n_mod) {
      if (pre > 0.f) {
        mode = kModeNone;
        p.a = 1.f;
        p.c2 = pre * kLog2eF;
      }
    } else if (a->mod_op[i] == LF_MOD_TANH) {
      int j = i + 1;
      float post = 1.f;
      while (j < a->n_mod && (a->mod_op[j] == LF_MOD_MUL || a->mod_op[j] == LF_MOD_DIV)) {
        post = a->mod_op[j] == LF_MOD_MUL ? post * a->mod_arg[j] : post / a->mod_arg[j];
        ++j;
      }
      if (j == a->n_mod && post > 0.f) {
        p.a = pre;
        p.c2 = post * kLog2eF;
        // |logit2| <= c2: small enough for the fixed softmax reference (the row sum of up to
        // 2^22 terms of at most 2^80 stays far below the fp32 limit).
        // (the fixed-reference kernels read dense K/V; a paged operand goes to the running-max
        // kernel, whose producer warp can gather)
        mode = (p.c2 <= kBoundedMaxC2 && a->Skv <= (1 << 22) && !p.paged) ? kModeBounded
                                                                           : kModeSoftcap;
        const float a2 = p.a * p.a, k0 = p.a * p.c2;
        p.qc[0] = k0;
        p.qc[1] = k0 * a2 * (-1.f / 3.f);
        p.qc[2] = k0 * a2 * a2 * (2.f / 15.f);
        p.qc[3] = k0 * a2 * a2 * a2 * (-17.f / 315.f);
        p.ylim[0] = kTanhPoly1Limit * kTanhPoly1Limit / a2;
        p.ylim[1] = kTanhPoly3Limit * kTanhPoly3Limit / a2;
      }
    }
  }
  {
    if (mode == kModeGeneric) {
      p.a = a->scale;
      p.c2 = kLog2eF;
      p.mods.n = a->n_mod;
      for (int m = 0; m < a->n_mod; ++m) {
        p.mods.op[m] = a->mod_op[m];
        p.mods.arg[m] = a->mod_arg[m];
      }
    }
  }

  if (has_pe) {
    // The two-product form runs in the plain running-max mode only (scale, then mask).
    if (mode == kModeBounded || mode == kModeSoftcap || mode == kModeGeneric)
      return LF_ERR_UNSUPPORTED;
  }
  const int kv_tile = choose_kv_tile(a, mode);
  if (kv_tile < 0) return kv_tile;
  // Two or four query heads per kv head under a window mask: the packed layout of the
  // fixed-reference kernel (128 / group query rows of each of the heads per tile slot).
  const int pack = (mode == kModeBounded && kv_tile != kWideK && (p.group == 2 || p.group == 4) &&
                    a->mask_kind == LF_MASK_CAUSAL_WINDOW) ? p.group : 1;
  if (q_tile) *q_tile = kTileQ / pack;
  if (launch == nullptr) return kv_tile;  // query only

  CUtensorMap mq, mk, mv;
  int rc = make_tile_map(&mq, a->q, a->B, a->Hq, a->Sq, a->D, a->q_stride, kTileQ / pack);
  if (rc != LF_OK) return rc;
  if (p.paged & 1) {
    mk = mq;  // never used: the producer warp gathers K itself
  } else {
    rc = make_tile_map(&mk, a->k, a->B, a->Hkv, a->Skv, a->D, a->k_stride, kv_tile);
    if (rc != LF_OK) return rc;
  }
  if (p.paged & 2) {
    mv = mq;
  } else {
    rc = make_tile_map(&mv, a->v, a->B, a->Hkv, a->Skv, a->D, a->v_stride, kv_tile);
    if (rc != LF_OK) return rc;
  }

  CUtensorMap mo;  // output store boxes of the persistent kernels: 32 rows x 32 columns
  if (mode == kModeBounded) {
    rc = make_tile_map(&mo, a->out, a->B, a->Hq, a->Sq, a->D, a->o_stride, 32,
                       (pack > 1 && a->D == 128) ? 64 : 32);
    if (rc != LF_OK) return rc;
  }

  cudaStream_t st = static_cast<cudaStream_t>(*launch);
  if (has_pe) {
    // Boxes of 64 columns over tensors of D_pe columns: the columns past D_pe arrive as zeros.
    CUtensorMap mqpe, mkpe;
    rc = make_tile_map(&mqpe, a->q_pe, a->B, a->Hq, a->Sq, a->D_pe, a->qpe_stride, kTileQ);
    if (rc != LF_OK) return rc;
    rc = make_tile_map(&mkpe, a->k_pe, a->B, a->Hkv, a->Skv, a->D_pe, a->kpe_stride, kTileK);
    if (rc != LF_OK) return rc;
    if (a->D == 128)
      return launch_prefill<128, kModeNone, true>(mq, mk, mv, p, a->B, st, &mqpe, &mkpe);
    return launch_prefill<64, kModeNone, true>(mq, mk, mv, p, a->B, st, &mqpe, &mkpe);
  }
  if (a->D == 128) {
    if (mode == kModeNone) return launch_prefill<128, kModeNone>(mq, mk, mv, p, a->B, st);
    if (mode == kModeSoftcap) return launch_prefill<128, kModeSoftcap>(mq, mk, mv, p, a->B, st);
    if (mode == kModeBounded)
      return kv_tile == kWideK ? launch_prefill_wide<128>(mq, mk, mv, mo, p, a->B, st)
             : pack == 4       ? launch_prefill_bounded<128, 4>(mq, mk, mv, mo, p, a->B, st)
             : pack == 2       ? launch_prefill_bounded<128, 2>(mq, mk, mv, mo, p, a->B, st)
                               : launch_prefill_bounded<128>(mq, mk, mv, mo, p, a->B, st);
    return launch_prefill<128, kModeGeneric>(mq, mk, mv, p, a->B, st);
  }
  if (mode == kModeNone) return launch_prefill<64, kModeNone>(mq, mk, mv, p, a->B, st);
  if (mode == kModeSoftcap) return launch_prefill<64, kModeSoftcap>(mq, mk, mv, p, a->B, st);
  if (mode == kModeBounded)
    return kv_tile == kWideK ? launch_prefill_wide<64>(mq, mk, mv, mo, p, a->B, st)
           : pack == 4       ? launch_prefill_bounded<64, 4>(mq, mk, mv, mo, p, a->B, st)
           : pack == 2       ? launch_prefill_bounded<64, 2>(mq, mk, mv, mo, p, a->B, st)
                             : launch_prefill_bounded<64>(mq, mk, mv, mo, p, a->B, st);
  return launch_prefill<64, kModeGeneric>(mq, mk, mv, p, a->B, st);
}

}  // namespace lf

extern "C" {

int lf_prefill_bf16(const LfPrefillArgs* args, void* stream) {
  return lf::prefill_impl(args, &stream);
}

int lf_prefill_kv_tile(const LfPrefillArgs* args) { return lf::prefill_impl(args, nullptr); }

int lf_prefill_q_tile(const LfPrefillArgs* args) {
  int q_tile = 0;
  const int rc = lf::prefill_impl(args, nullptr, &q_tile);
  return rc < 0 ? rc : q_tile;
}

void lf_tile_map_cache_stats(uint64_t* hits, uint64_t* misses) {
  if (hits) *hits = lf::g_tile_map_hits.load();
  if (misses) *misses = lf::g_tile_map_misses.load();
}

void lf_skip_range(int32_t mask_kind, int32_t window, int32_t causal_offset, int32_t Sq,
                   int32_t Skv, int32_t tile_q, int32_t tile_k, int32_t iq, int32_t* lo,
                   int32_t* hi) {
  lf::skip_range(mask_kind, window, causal_offset, Sq, Skv, tile_q, tile_k, iq, lo, hi);
}

}  // extern "C"
