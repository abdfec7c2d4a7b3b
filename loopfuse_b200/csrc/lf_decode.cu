// Decode attention for sm_100a: one query row per head, KV streamed once from HBM.
//
// Bandwidth-bound, so the work is laid out to keep many 16-byte loads in flight:
//   * a CTA owns one (batch, kv head, KV split); its 4 warps interleave over the tokens of
//     the split, each thread issuing UNROLL K-row and UNROLL V-row 16-byte streaming loads
//     before any arithmetic;
//   * a K/V row of D bf16 is covered by D/8 lanes, so a warp reads 32/(D/8) whole rows per
//     load instruction (fully used 32-byte sectors);
//   * the G query heads that share the kv head are kept in registers and reuse every loaded
//     row (GQA), scores are reduced with shuffles, softmax is online in the log2 domain;
//   * with splits > 1 each CTA writes an un-normalised partial (acc, max, sum) to the
//     workspace and lf_combine merges them (log-sum-exp combine);
//   * the paged variant stages its slice of the block table through shared memory, checks
//     every page id against the pool size (status word, clamped, never a trap) and turns
//     (page, slot) into row pointers.
#include "lf_common.cuh"

#include <math.h>

#include <mutex>

namespace lf {

constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kDecodeUnroll = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kMmaStages = 3;  // cp.async ring depth of the tensor-core decode kernel

struct DecodeParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  __nv_bfloat16* out;
  float* part_o;   // [units, splits, D]
  float* part_ml;  // [units, splits, 2]
  const int32_t* block_table;
  const int32_t* block_table_v;  // never null for the paged kernel (may equal block_table)
  int32_t* status;
  int64_t q_stride[3], o_stride[3], k_stride[3], v_stride[3];
  int64_t bt_stride;
  int32_t B, Hkv, Skv, splits, chunk;  // chunk = tokens per split
  int32_t page_size, page_shift, n_pages;  // page_shift >= 0 when page_size is 2^shift
  float scale;
  ModChain mods;
};

template <int D, int G, bool PAGED, bool HAS_MOD>
__global__ void __launch_bounds__(kDecodeThreads)
    decode_split_kernel(const DecodeParams p) {
  constexpr int LPR = D / 8;        // lanes per K/V row
  constexpr int RPW = 32 / LPR;     // rows per warp-wide load
  constexpr int U = kDecodeUnroll;  // rows in flight per thread and tensor
  constexpr int TOK_PER_WARP_IT = U * RPW;
  constexpr int TOK_PER_CTA_IT = TOK_PER_WARP_IT * kDecodeWarps;

  const int split = blockIdx.x;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rg = lane / LPR;   // row group inside the warp
  const int col = lane % LPR;  // which 8-element slice of the row

  const int t0 = split * p.chunk;
  const int t1 = min(p.Skv, t0 + p.chunk);

  extern __shared__ __align__(16) unsigned char smem_raw[];
  // Layout: [page ids of this split] (paged only), then the cross-warp merge area.
  int32_t* s_pages_k = reinterpret_cast<int32_t*>(smem_raw);
  int32_t* s_pages_v = s_pages_k;
  int n_pages_local = 0;
  int first_page = 0;
  size_t merge_off = 0;
  if constexpr (PAGED) {
    auto page_of = [&](int t) { return p.page_shift >= 0 ? (t >> p.page_shift) : (t / p.page_size); };
    if (t1 > t0) {
      first_page = page_of(t0);
      n_pages_local = page_of(t1 - 1) - first_page + 1;
    }
    const bool two_tables = p.block_table_v != p.block_table;
    const int pages_pad = (n_pages_local + 3) & ~3;
    if (two_tables) s_pages_v = s_pages_k + pages_pad;
    merge_off = static_cast<size_t>(pages_pad) * 4 * (two_tables ? 2 : 1);
    for (int which = 0; which < (two_tables ? 2 : 1); ++which) {
      const int32_t* bt = (which == 0 ? p.block_table : p.block_table_v) +
                          static_cast<int64_t>(b) * p.bt_stride + first_page;
      int32_t* dst = which == 0 ? s_pages_k : s_pages_v;
      for (int i = threadIdx.x; i < n_pages_local; i += kDecodeThreads) {
        int32_t pg = bt[i];
        if (pg < 0 || pg >= p.n_pages) {
          if (p.status) atomicExch(p.status, LF_DEV_BAD_PAGE);
          pg = 0;
        }
        dst[i] = pg;
      }
    }
    __syncthreads();
  }
  float* s_merge = reinterpret_cast<float*>(smem_raw + merge_off);

  // Query rows for the G grouped heads, this lane's 8-element slice, as fp32. Without a
  // score-mod chain the softmax scale and log2(e) are folded into q.
  float qf[G][8];
  {
    const float qmul = HAS_MOD ? p.scale : p.scale * kLog2e;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const __nv_bfloat16* qp =
          p.q + b * p.q_stride[0] + kvh * p.q_stride[1] + g * p.q_stride[2] + col * 8;
      const uint4 raw = *reinterpret_cast<const uint4*>(qp);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        qf[g][2 * i] = bf16lo_to_f32(w[i]) * qmul;
        qf[g][2 * i + 1] = bf16hi_to_f32(w[i]) * qmul;
      }
    }
  }

  float m_run[G], l_run[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  }

  const __nv_bfloat16* kbase;
  const __nv_bfloat16* vbase;
  if constexpr (PAGED) {
    kbase = p.k + kvh * p.k_stride[2] + col * 8;
    vbase = p.v + kvh * p.v_stride[2] + col * 8;
  } else {
    kbase = p.k + b * p.k_stride[0] + kvh * p.k_stride[1] + col * 8;
    vbase = p.v + b * p.v_stride[0] + kvh * p.v_stride[1] + col * 8;
  }

  for (int base = t0 + warp * TOK_PER_WARP_IT; base < t1; base += TOK_PER_CTA_IT) {
    uint4 kr[U], vr[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = base + u * RPW + rg;
      valid[u] = t < t1;
      int tc = valid[u] ? t : (t1 - 1);  // clamp: the row is loaded but scored -inf
      if (!LF_BOUNDS(tc >= t0 && tc < p.Skv, p.status, 40)) tc = t0;
      int64_t koff, voff;
      if constexpr (PAGED) {
        const int pg_abs = p.page_shift >= 0 ? (tc >> p.page_shift) : (tc / p.page_size);
        const int slot = tc - pg_abs * p.page_size;
        int pl = pg_abs - first_page;
        if (!LF_BOUNDS(pl >= 0 && pl < n_pages_local && slot >= 0 && slot < p.page_size,
                       p.status, 41))
          pl = 0;
        const int64_t pgk = s_pages_k[pl];
        const int64_t pgv = s_pages_v[pl];
        koff = pgk * p.k_stride[0] + slot * p.k_stride[1];
        voff = pgv * p.v_stride[0] + slot * p.v_stride[1];
      } else {
        koff = tc * p.k_stride[2];
        voff = tc * p.v_stride[2];
      }
      kr[u] = ldg_stream_16(kbase + koff);
      vr[u] = ldg_stream_16(vbase + voff);
    }

    // Scores: partial dot over this lane's 8 elements, then all-reduce over the row's lanes.
    float s[G][U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t w[4] = {kr[u].x, kr[u].y, kr[u].z, kr[u].w};
      float kf[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        kf[2 * i] = bf16lo_to_f32(w[i]);
        kf[2 * i + 1] = bf16hi_to_f32(w[i]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(qf[g][e], kf[e], d);
        s[g][u] = d;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float d = s[g][u];
#pragma unroll
        for (int off = LPR / 2; off >= 1; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        if constexpr (HAS_MOD) d = apply_mods(p.mods, d) * kLog2e;
        s[g][u] = valid[u] ? d : -INFINITY;
      }
    }

    // Online softmax update (log2 domain) and PV accumulation.
    float pw[G][U];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float m_new = m_run[g];
#pragma unroll
      for (int u = 0; u < U; ++u) m_new = fmaxf(m_new, s[g][u]);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = ex2_approx(m_run[g] - m_safe);
      float psum = 0.f;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        pw[g][u] = ex2_approx(s[g][u] - m_safe);
        psum += pw[g][u];
      }
      l_run[g] = l_run[g] * alpha + psum;
      m_run[g] = m_new;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= alpha;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t w[4] = {vr[u].x, vr[u].y, vr[u].z, vr[u].w};
      float vf[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        vf[2 * i] = bf16lo_to_f32(w[i]);
        vf[2 * i + 1] = bf16hi_to_f32(w[i]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pw[g][u], vf[e], acc[g][e]);
      }
    }
  }

  // Merge the row groups of a warp (they hold disjoint token subsets of the same columns).
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m_run[g], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l_run[g], off);
      const float m_new = fmaxf(m_run[g], m_o);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float a_s = ex2_approx(m_run[g] - m_safe);
      const float a_o = ex2_approx(m_o - m_safe);
      l_run[g] = l_run[g] * a_s + l_o * a_o;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float acc_o = __shfl_xor_sync(0xffffffffu, acc[g][e], off);
        acc[g][e] = acc[g][e] * a_s + acc_o * a_o;
      }
      m_run[g] = m_new;
    }
  }

  // Merge the warps through shared memory: s_merge[warp][g][0..D) acc, then m, l.
  constexpr int kStride = D + 2;
  if (rg == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* dst = s_merge + (warp * G + g) * kStride;
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[col * 8 + e] = acc[g][e];
      if (col == 0) {
        dst[D] = m_run[g];
        dst[D + 1] = l_run[g];
      }
    }
  }
  __syncthreads();

  // One thread per (g, column) finishes the merge and writes the result.
  for (int idx = threadIdx.x; idx < G * D; idx += kDecodeThreads) {
    const int g = idx / D;
    const int c = idx - g * D;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w)
      m_all = fmaxf(m_all, s_merge[(w * G + g) * kStride + D]);
    const float m_safe = (m_all == -INFINITY) ? 0.f : m_all;
    float l_all = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float* src = s_merge + (w * G + g) * kStride;
      const float a = ex2_approx(src[D] - m_safe);
      l_all += src[D + 1] * a;
      o += src[c] * a;
    }
    const int64_t unit = (static_cast<int64_t>(b) * p.Hkv + kvh) * G + g;
    if (p.splits == 1) {
      __nv_bfloat16* op = p.out + b * p.o_stride[0] + kvh * p.o_stride[1] + g * p.o_stride[2];
      op[c] = __float2bfloat16_rn(o / l_all);
    } else {
      p.part_o[(unit * p.splits + split) * D + c] = o;
      if (c == 0) {
        p.part_ml[(unit * p.splits + split) * 2] = m_all;
        p.part_ml[(unit * p.splits + split) * 2 + 1] = l_all;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Grouped / paged decode on tensor cores (mma.sync m16n8k16, bf16 -> fp32).
//
// For G > 2 query rows per kv head (and for every paged cache) the FMA + shuffle form above
// becomes instruction-bound long before HBM is saturated; here the G rows are the (zero-padded)
// M dimension of 16x8x16 MMAs and the fragments come straight from 16-byte global loads:
//
//   QK^T  8 tokens at a time. Lane (n = lane/4, c = lane%4) loads the 16-byte pieces
//         d = 32i + 8c .. +8 of token n's K row (i < D/32); the four 32-bit words of a piece
//         are exactly the B fragments of two MMAs (a dot product does not care in which order
//         the d's are visited as long as Q uses the same order, and Q is loaded with the same
//         pattern, row g = lane/4 instead of token n).
//   PV    16 tokens at a time. Lane (n, c) loads rows 2c, 2c+1, 2c+8, 2c+9 at d = 64h + 8n ..
//         +8; a byte permute of two rows gives the {V[2c][d], V[2c+1][d]} pairs the B fragment
//         wants; output column n of MMA (h, e) stands for d = 64h + 8n + e.
//   The fp32 score fragment of the QK MMAs has the layout of the bf16 A fragment of the PV
//   MMA, so P never leaves registers.
// A CTA is one (batch, kv head, KV split); its WARPS warps (4, or 2 when smaller CTAs let the
// whole grid be resident at once) take alternate 16-token groups (one page when page_size is
// 16) and are merged through shared memory like above.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_16816_rows0to7(float& d0, float& d1, uint32_t a0, uint32_t a2,
                                                   uint32_t b0, uint32_t b1) {
  [[maybe_unused]] float unused2, unused3;  // rows 8..15 of the tile are padding
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %10, %11};"
      : "+f"(d0), "+f"(d1), "=f"(unused2), "=f"(unused3)
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f), "f"(0.f));
}

template <int D, bool PAGED, bool HAS_MOD, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 12 / WARPS)
    decode_mma_kernel(const DecodeParams p, const int G) {
  constexpr int KI = D / 32;  // 16-byte pieces of a K row per lane
  constexpr int VH = D / 64;  // 64-wide halves of a V row
  constexpr int NT = D / 8;   // output n-tiles (8 columns each)

  const int split = blockIdx.x;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;  // query row of this lane's score / output fragment; token index n
  const int c = lane & 3;

  const int t0 = split * p.chunk;
  const int t1 = min(p.Skv, t0 + p.chunk);

  extern __shared__ __align__(16) unsigned char smem_raw[];
  int32_t* s_pages_k = reinterpret_cast<int32_t*>(smem_raw);
  int32_t* s_pages_v = s_pages_k;
  int first_page = 0;
  size_t merge_off = 0;
  auto page_of = [&](int t) { return p.page_shift >= 0 ? (t >> p.page_shift) : (t / p.page_size); };
  if constexpr (PAGED) {
    int n_pages_local = 0;
    if (t1 > t0) {
      first_page = page_of(t0);
      n_pages_local = page_of(t1 - 1) - first_page + 1;
    }
    const bool two_tables = p.block_table_v != p.block_table;
    const int pages_pad = (n_pages_local + 3) & ~3;
    if (two_tables) s_pages_v = s_pages_k + pages_pad;
    merge_off = static_cast<size_t>(pages_pad) * 4 * (two_tables ? 2 : 1);
    for (int which = 0; which < (two_tables ? 2 : 1); ++which) {
      const int32_t* bt = (which == 0 ? p.block_table : p.block_table_v) +
                          static_cast<int64_t>(b) * p.bt_stride + first_page;
      int32_t* dst = which == 0 ? s_pages_k : s_pages_v;
      for (int i = threadIdx.x; i < n_pages_local; i += (WARPS * 32)) {
        int32_t pg = bt[i];
        if (pg < 0 || pg >= p.n_pages) {
          if (p.status) atomicExch(p.status, LF_DEV_BAD_PAGE);
          pg = 0;
        }
        dst[i] = pg;
      }
    }
    __syncthreads();
  }
  float* s_merge = reinterpret_cast<float*>(smem_raw + merge_off);

  // Row pointers of token t for this lane's kv head.
  const __nv_bfloat16* kbase;
  const __nv_bfloat16* vbase;
  if constexpr (PAGED) {
    kbase = p.k + kvh * p.k_stride[2];
    vbase = p.v + kvh * p.v_stride[2];
  } else {
    kbase = p.k + b * p.k_stride[0] + kvh * p.k_stride[1];
    vbase = p.v + b * p.v_stride[0] + kvh * p.v_stride[1];
  }
  [[maybe_unused]] const int n_pages_staged =
      (PAGED && t1 > t0) ? page_of(t1 - 1) - first_page + 1 : 0;
  auto k_row = [&](int t) -> const __nv_bfloat16* {
    if (!LF_BOUNDS(t >= t0 && t < t1 && t < p.Skv, p.status, 42)) t = t0;
    if constexpr (PAGED) {
      const int pg_abs = page_of(t);
      const int slot = t - pg_abs * p.page_size;
      if (!LF_BOUNDS(pg_abs - first_page >= 0 && pg_abs - first_page < n_pages_staged,
                     p.status, 43))
        return kbase;
      return kbase + static_cast<int64_t>(s_pages_k[pg_abs - first_page]) * p.k_stride[0] +
             slot * p.k_stride[1];
    } else {
      return kbase + t * p.k_stride[2];
    }
  };
  auto v_row = [&](int t) -> const __nv_bfloat16* {
    if (!LF_BOUNDS(t >= t0 && t < t1 && t < p.Skv, p.status, 44)) t = t0;
    if constexpr (PAGED) {
      const int pg_abs = page_of(t);
      const int slot = t - pg_abs * p.page_size;
      if (!LF_BOUNDS(pg_abs - first_page >= 0 && pg_abs - first_page < n_pages_staged,
                     p.status, 45))
        return vbase;
      return vbase + static_cast<int64_t>(s_pages_v[pg_abs - first_page]) * p.v_stride[0] +
             slot * p.v_stride[1];
    } else {
      return vbase + t * p.v_stride[2];
    }
  };

  // Q fragments (rows g >= G are zero padding).
  uint4 qr[KI];
#pragma unroll
  for (int i = 0; i < KI; ++i) {
    qr[i] = make_uint4(0u, 0u, 0u, 0u);
    if (g < G)
      qr[i] = *reinterpret_cast<const uint4*>(p.q + b * p.q_stride[0] + kvh * p.q_stride[1] +
                                              g * p.q_stride[2] + 32 * i + 8 * c);
  }
  const float smul = HAS_MOD ? p.scale : p.scale * kLog2e;

  float m_run = -INFINITY, l_run = 0.f;
  float o[NT][2];
#pragma unroll
  for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = 0.f;

  // K/V rows travel global -> shared with 16-byte cp.async into a ring private to the warp
  // (kMmaStages groups of 16 tokens; kMmaStages-1 groups are in flight while one is consumed),
  // so the bytes in flight do not cost registers. A 16-byte chunk j of row r sits at chunk
  // position j ^ (r & 7): fragment reads of eight different rows then hit distinct banks.
  constexpr int CPR = D / 8;               // 16-byte chunks per row
  constexpr int kRowBytes = D * 2;
  constexpr int kStageBytes = 2 * 16 * kRowBytes;  // 16 K rows then 16 V rows
  const int t_last = t1 - 1;
  unsigned char* ring = smem_raw + merge_off + warp * (kMmaStages * kStageBytes);
  const uint32_t ring_u32 = smem_u32(ring);
  auto copy_group = [&](int tg, int stage) {
    if (tg < t1) {
      const uint32_t dst0 = ring_u32 + stage * kStageBytes;
      const int j = lane % CPR;
      const int r_max = t_last - tg;  // rows past the end of the split re-read the last token
      // A group that lies inside one page (always true for dense caches) has affine row
      // addresses: one table lookup per group instead of one per row.
      bool one_page = true;
      if constexpr (PAGED) one_page = page_of(tg) == page_of(min(tg + 15, t_last));
      if (one_page) {
        const __nv_bfloat16* kp = k_row(tg) + 8 * j;
        const __nv_bfloat16* vp = v_row(tg) + 8 * j;
        const int64_t ks = PAGED ? p.k_stride[1] : p.k_stride[2];
        const int64_t vs = PAGED ? p.v_stride[1] : p.v_stride[2];
#pragma unroll
        for (int q = 0; q < 16 * CPR / 32; ++q) {
          const int r = lane / CPR + q * (32 / CPR);
          const int rc = min(r, r_max);
          const uint32_t off = r * kRowBytes + ((j ^ (r & 7)) << 4);
          if (!LF_BOUNDS(off + 16 <= 16u * kRowBytes && stage >= 0 && stage < kMmaStages,
                         p.status, 46))
            continue;
          cp_async_16(dst0 + off, kp + rc * ks);
          cp_async_16(dst0 + 16 * kRowBytes + off, vp + rc * vs);
        }
      } else {
#pragma unroll
        for (int q = 0; q < 16 * CPR / 32; ++q) {
          const int r = lane / CPR + q * (32 / CPR);
          const int tok = tg + min(r, r_max);
          const uint32_t off = r * kRowBytes + ((j ^ (r & 7)) << 4);
          cp_async_16(dst0 + off, k_row(tok) + 8 * j);
          cp_async_16(dst0 + 16 * kRowBytes + off, v_row(tok) + 8 * j);
        }
      }
    }
    cp_async_commit();
  };
  const int tg0 = t0 + warp * 16;
#pragma unroll
  for (int st = 0; st < kMmaStages - 1; ++st) copy_group(tg0 + st * 16 * WARPS, st);

  int it = 0;
  for (int tg = tg0; tg < t1; tg += 16 * WARPS, ++it) {
    copy_group(tg + (kMmaStages - 1) * 16 * WARPS, (it + kMmaStages - 1) % kMmaStages);
    cp_async_wait<kMmaStages - 1>();
    __syncwarp();
    const unsigned char* stage = ring + (it % kMmaStages) * kStageBytes;
    // K: token n = g of each 8-token half; V: rows 2c, 2c+1, 2c+8, 2c+9 of the 16-token group.
    uint4 kr[2][KI];
#pragma unroll
    for (int s8 = 0; s8 < 2; ++s8) {
      const int r = 8 * s8 + g;
#pragma unroll
      for (int i = 0; i < KI; ++i)
        kr[s8][i] = *reinterpret_cast<const uint4*>(stage + r * kRowBytes +
                                                    (((4 * i + c) ^ (r & 7)) << 4));
    }

    // Scores of the two 8-token halves: this lane ends up with tokens 2c, 2c+1 of each.
    float sc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int s8 = 0; s8 < 2; ++s8)
#pragma unroll
      for (int i = 0; i < KI; ++i) {
        mma_16816_rows0to7(sc[s8][0], sc[s8][1], qr[i].x, qr[i].y, kr[s8][i].x, kr[s8][i].y);
        mma_16816_rows0to7(sc[s8][0], sc[s8][1], qr[i].z, qr[i].w, kr[s8][i].z, kr[s8][i].w);
      }
    float mx = -INFINITY;
#pragma unroll
    for (int s8 = 0; s8 < 2; ++s8)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float v = sc[s8][e] * smul;
        if constexpr (HAS_MOD) v = apply_mods(p.mods, v) * kLog2e;
        if (tg + 8 * s8 + 2 * c + e >= t1) v = -INFINITY;
        sc[s8][e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = ex2_approx(m_run - m_safe);
    m_run = m_new;
    float pr[2][2];
    float psum = 0.f;
#pragma unroll
    for (int s8 = 0; s8 < 2; ++s8)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pr[s8][e] = ex2_approx(sc[s8][e] - m_safe);
        psum += pr[s8][e];
      }
    l_run = l_run * alpha + psum;  // this lane's share; the quad is summed after the loop
    const uint32_t pa0 = pack_bf16x2(pr[0][0], pr[0][1]);
    const uint32_t pa2 = pack_bf16x2(pr[1][0], pr[1][1]);
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      o[j][0] *= alpha;
      o[j][1] *= alpha;
    }
#pragma unroll
    for (int h = 0; h < VH; ++h) {
      uint4 vq[4];
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int r = 2 * c + (r4 & 1) + 8 * (r4 >> 1);
        vq[r4] = *reinterpret_cast<const uint4*>(stage + (16 + r) * kRowBytes +
                                                 (((8 * h + g) ^ (r & 7)) << 4));
      }
      const uint32_t w0[4] = {vq[0].x, vq[0].y, vq[0].z, vq[0].w};
      const uint32_t w1[4] = {vq[1].x, vq[1].y, vq[1].z, vq[1].w};
      const uint32_t w2[4] = {vq[2].x, vq[2].y, vq[2].z, vq[2].w};
      const uint32_t w3[4] = {vq[3].x, vq[3].y, vq[3].z, vq[3].w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;  // high or low halves of two words
        const uint32_t b0 = __byte_perm(w0[e >> 1], w1[e >> 1], sel);
        const uint32_t b1 = __byte_perm(w2[e >> 1], w3[e >> 1], sel);
        mma_16816_rows0to7(o[h * 8 + e][0], o[h * 8 + e][1], pa0, pa2, b0, b1);
      }
    }
    __syncwarp();  // every lane is done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // Row sum over the quad (the four lanes of a row hold disjoint tokens).
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

  // Merge the warps through shared memory: s_merge[warp][g][0..D) acc, then m, l. The merge
  // area reuses the rings, so every warp must have finished reading its last stage.
  constexpr int kStride = D + 2;
  __syncthreads();
  if (g < G) {
    float* dst = s_merge + (warp * G + g) * kStride;
#pragma unroll
    for (int h = 0; h < VH; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dst[64 * h + 16 * c + e] = o[h * 8 + e][0];      // output column 2c   -> d = 64h+16c+e
        dst[64 * h + 16 * c + 8 + e] = o[h * 8 + e][1];  // output column 2c+1 -> d + 8
      }
    if (c == 0) {
      dst[D] = m_run;
      dst[D + 1] = l_run;
    }
  }
  __syncthreads();

  for (int idx = threadIdx.x; idx < G * D; idx += (WARPS * 32)) {
    const int gg = idx / D;
    const int cc = idx - gg * D;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w)
      m_all = fmaxf(m_all, s_merge[(w * G + gg) * kStride + D]);
    const float m_safe = (m_all == -INFINITY) ? 0.f : m_all;
    float l_all = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float* src = s_merge + (w * G + gg) * kStride;
      const float a = ex2_approx(src[D] - m_safe);
      l_all += src[D + 1] * a;
      acc += src[cc] * a;
    }
    const int64_t unit = (static_cast<int64_t>(b) * p.Hkv + kvh) * G + gg;
    if (!LF_BOUNDS(gg < G && cc < D && b < p.B && kvh < p.Hkv && split < p.splits, p.status, 47))
      continue;
    if (p.splits == 1) {
      __nv_bfloat16* op = p.out + b * p.o_stride[0] + kvh * p.o_stride[1] + gg * p.o_stride[2];
      op[cc] = __float2bfloat16_rn(acc / l_all);
    } else {
      p.part_o[(unit * p.splits + split) * D + cc] = acc;
      if (cc == 0) {
        p.part_ml[(unit * p.splits + split) * 2] = m_all;
        p.part_ml[(unit * p.splits + split) * 2 + 1] = l_all;
      }
    }
  }
}

// Log-sum-exp combine of split-KV partials: one warp per (batch, kv head, g) output row.
template <int D>
__global__ void __launch_bounds__(128)
    combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                   __nv_bfloat16* __restrict__ out, int64_t units, int32_t Hkv, int32_t G,
                   int32_t splits, int64_t os0, int64_t os1, int64_t os2) {
  constexpr int EPL = D / 32;  // elements per lane
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= units) return;
  // Lane s owns split s (at most 32 splits): one load round for all (max, sum) pairs, the
  // weights are then broadcast from their lanes while the partial rows stream in.
  const float* ml = part_ml + unit * splits * 2;
  float m_s = -INFINITY, l_s = 0.f;
  if (lane < splits) {
    const float2 v = *reinterpret_cast<const float2*>(ml + 2 * lane);
    m_s = v.x;
    l_s = v.y;
  }
  float m_all = m_s;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1)
    m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, off));
  const float m_safe = (m_all == -INFINITY) ? 0.f : m_all;
  const float w_s = ex2_approx(m_s - m_safe);
  float l_all = l_s * w_s;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) l_all += __shfl_xor_sync(0xffffffffu, l_all, off);
  float o[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) o[e] = 0.f;
  const float* src0 = part_o + unit * splits * D + lane * EPL;
  for (int s0 = 0; s0 < splits; s0 += 4) {
    float x[4][EPL];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int s = min(s0 + u, splits - 1);
      if constexpr (EPL == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src0 + s * D);
        x[u][0] = v.x; x[u][1] = v.y; x[u][2] = v.z; x[u][3] = v.w;
      } else {
        const float2 v = *reinterpret_cast<const float2*>(src0 + s * D);
        x[u][0] = v.x; x[u][1] = v.y;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float a = (s0 + u < splits) ? __shfl_sync(0xffffffffu, w_s, (s0 + u) & 31) : 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] += x[u][e] * a;
    }
  }
  const float inv = 1.f / l_all;
  const int64_t g = unit % G;
  const int64_t h = (unit / G) % Hkv;
  const int64_t bb = unit / G / Hkv;
  __nv_bfloat16* op = out + bb * os0 + h * os1 + g * os2 + lane * EPL;
  if constexpr (EPL == 4) {
    uint2 w;
    w.x = pack_bf16x2(o[0] * inv, o[1] * inv);
    w.y = pack_bf16x2(o[2] * inv, o[3] * inv);
    *reinterpret_cast<uint2*>(op) = w;
  } else {
    *reinterpret_cast<uint32_t*>(op) = pack_bf16x2(o[0] * inv, o[1] * inv);
  }
}

// out[b, h, t, :] = pool[block_table[b, t / P], t % P, h, :]; one warp-row group per token.
template <int D>
__global__ void __launch_bounds__(256)
    paged_gather_kernel(const __nv_bfloat16* __restrict__ pool,
                        const int32_t* __restrict__ block_table, __nv_bfloat16* __restrict__ out,
                        int32_t B, int32_t Hkv, int32_t Skv, int32_t page_size, int32_t n_pages,
                        int64_t ps0, int64_t ps1, int64_t ps2, int64_t bt_stride,
                        int32_t* status) {
  constexpr int LPR = D / 8;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  const int64_t row = gid / LPR;
  const int col = static_cast<int>(gid % LPR);
  const int64_t total_rows = static_cast<int64_t>(B) * Hkv * Skv;
  if (row >= total_rows) return;
  const int t = static_cast<int>(row % Skv);
  const int h = static_cast<int>((row / Skv) % Hkv);
  const int b = static_cast<int>(row / Skv / Hkv);
  int32_t pg = block_table[b * bt_stride + t / page_size];
  if (pg < 0 || pg >= n_pages) {
    if (status) atomicExch(status, LF_DEV_BAD_PAGE);
    pg = 0;
  }
  const int slot = t % page_size;
  const uint4 x = *reinterpret_cast<const uint4*>(pool + pg * ps0 + slot * ps1 + h * ps2 + col * 8);
  *reinterpret_cast<uint4*>(out + row * D + col * 8) = x;
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
static int device_sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    cached_dev = dev;
  }
  return cached > 0 ? cached : 148;
}

static int round_up(int x, int m) { return (x + m - 1) / m * m; }

static bool uses_mma_kernel(int G, bool paged) { return paged || G > 2; }

// Shared memory the tensor-core kernel may spend on block-table slices (both tables), so that
// two CTAs (K/V rings of 96 KB each at D = 128) still fit on one SM.
constexpr size_t kMaxTableBytes = 16 * 1024;

static size_t table_smem_bytes(int chunk, int page_size) {
  // Room for the K table and a separate V table, each padded to 16 bytes.
  return 2 * (((static_cast<size_t>(chunk / page_size) + 2 + 3) & ~size_t(3)) * 4);
}

// Largest token chunk of one split whose block-table slice fits (paged caches only).
static int max_chunk_for_table(int page_size) {
  const int entries = static_cast<int>(kMaxTableBytes / 8) - 4;  // per table, minus padding
  const int64_t tokens = static_cast<int64_t>(entries) * page_size;
  return static_cast<int>(tokens > (1 << 30) ? (1 << 30) : tokens / 64 * 64);
}

// Split count for splits == 0. page_size: 0 for a dense cache, else the tokens per page.
static int choose_splits(int B, int Hkv, int G, int Skv, int D, int page_size) {
  (void)D;
  const bool paged = page_size > 0;
  const int units = B * Hkv;
  const int sms = device_sm_count();
  int max_by_len = Skv / 256;  // keep >= 256 tokens per split
  if (max_by_len < 1) max_by_len = 1;
  if (max_by_len > 32) max_by_len = 32;
  int s;
  if (uses_mma_kernel(G, paged)) {
    // Two CTAs of the tensor-core kernel are resident per SM and each keeps ~16 KB in flight
    // per warp, so one wave already saturates HBM: split only to fill the machine (splitting
    // costs the partial round trip and a short, badly pipelined loop per CTA; splitting four
    // ways to even out the waves of 512 units measured 20 % slower than not splitting).
    const int resident = sms * 2;
    s = units >= resident ? 1 : (resident + units - 1) / units;
  } else {
    // The FMA kernel has ~8 small CTAs per SM: aim for >= 6 waves so the tail wave is cheap.
    s = (sms * 8 * 6 + units - 1) / units;
  }
  if (s > max_by_len) s = max_by_len;
  if (s < 1) s = 1;
  if (paged) {
    // The block-table slice of a split must fit in shared memory (one-token pages at long
    // context): split further until it does.
    const int max_chunk = max_chunk_for_table(page_size);
    while (s < 32 && round_up((Skv + s - 1) / s, 64) > max_chunk) ++s;
  }
  return s;
}

template <int D, int G, bool PAGED>
static int launch_decode_g(const DecodeParams& p, cudaStream_t st, size_t smem) {
  dim3 grid(p.splits, p.Hkv, p.B);
  if (p.mods.n > 0)
    decode_split_kernel<D, G, PAGED, true><<<grid, kDecodeThreads, smem, st>>>(p);
  else
    decode_split_kernel<D, G, PAGED, false><<<grid, kDecodeThreads, smem, st>>>(p);
  return check_launch("decode_split_kernel");
}

// Warps per CTA of the tensor-core kernel. Four warps (two CTAs resident per SM, K/V rings of
// 96 KB each at D = 128) by default. When the grid is more than one wave of such CTAs but fits
// in one wave of half-sized ones (four resident per SM, same bytes in flight per SM), two warps:
// 512 CTAs on 148 SMs are 1.73 waves of the large shape, whose second wave leaves a quarter of
// the machine idle, but a single resident grid of the small one.
static int mma_warps_per_cta(int64_t ctas) {
  const int sms = device_sm_count();
  return (ctas > 2ll * sms && ctas <= 4ll * sms) ? 2 : 4;
}

template <int D, bool PAGED, bool HAS_MOD, int WARPS>
static int launch_decode_mma_w(const DecodeParams& p, int G, cudaStream_t st, size_t table_bytes) {
  dim3 grid(p.splits, p.Hkv, p.B);
  // page ids + the per-warp K/V rings (the warp-merge area reuses the rings)
  const size_t ring = static_cast<size_t>(WARPS) * kMmaStages * 2 * 16 * D * 2;
  const size_t merge = static_cast<size_t>(WARPS) * G * (D + 2) * sizeof(float);
  const size_t smem = table_bytes + (ring > merge ? ring : merge);
  static thread_local int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<D, PAGED, HAS_MOD, WARPS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) {
      set_cuda_error(e, "cudaFuncSetAttribute(decode_mma_kernel)");
      return LF_ERR_CUDA;
    }
    configured_dev = dev;
  }
  decode_mma_kernel<D, PAGED, HAS_MOD, WARPS><<<grid, WARPS * 32, smem, st>>>(p, G);
  return check_launch("decode_mma_kernel");
}

template <int D, bool PAGED>
static int launch_decode_mma(const DecodeParams& p, int G, cudaStream_t st, size_t smem) {
  // `smem` arrives as warp-merge area (sized for four warps) + block-table slices.
  const size_t table_bytes = smem - static_cast<size_t>(kDecodeWarps) * G * (D + 2) * sizeof(float);
  const int warps = mma_warps_per_cta(static_cast<int64_t>(p.splits) * p.Hkv * p.B);
  if (p.mods.n > 0) {
    return warps == 2 ? launch_decode_mma_w<D, PAGED, true, 2>(p, G, st, table_bytes)
                      : launch_decode_mma_w<D, PAGED, true, 4>(p, G, st, table_bytes);
  }
  return warps == 2 ? launch_decode_mma_w<D, PAGED, false, 2>(p, G, st, table_bytes)
                    : launch_decode_mma_w<D, PAGED, false, 4>(p, G, st, table_bytes);
}

// Dense caches with one or two query rows per kv head stay on the FMA kernel (it already
// streams at HBM speed there); everything else runs on the tensor-core kernel.
template <int D, bool PAGED>
static int launch_decode(const DecodeParams& p, int G, cudaStream_t st, size_t smem) {
  if (uses_mma_kernel(G, PAGED)) return launch_decode_mma<D, PAGED>(p, G, st, smem);
  switch (G) {
    case 1: return launch_decode_g<D, 1, PAGED>(p, st, smem);
    case 2: return launch_decode_g<D, 2, PAGED>(p, st, smem);
    default: return LF_ERR_UNSUPPORTED;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int decode_impl(const LfDecodeArgs* a, void* stream, bool paged) {
  if (!a || !a->q || !a->k || !a->v || !a->out) return LF_ERR_INVALID_ARG;
  if (a->B <= 0 || a->Hkv <= 0 || a->G <= 0 || a->Skv <= 0) return LF_ERR_INVALID_ARG;
  if (a->D != 64 && a->D != 128) return LF_ERR_UNSUPPORTED;
  if (a->G != 1 && a->G != 2 && a->G != 4 && a->G != 8) return LF_ERR_UNSUPPORTED;
  if (a->n_mod < 0 || a->n_mod > LF_MAX_MODS) return LF_ERR_INVALID_ARG;
  if (a->Hkv > 65535 || a->B > 65535) return LF_ERR_TOO_LARGE;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out))
    return LF_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i) {
    if ((a->q_stride[i] % 8) || (a->k_stride[i] % 8) || (a->v_stride[i] % 8) ||
        (a->o_stride[i] % 4))
      return LF_ERR_ALIGNMENT;
  }
  if (paged) {
    if (!a->block_table || a->page_size <= 0 || a->n_pages <= 0) return LF_ERR_INVALID_ARG;
  }
  int splits = a->splits;
  if (splits < 0) return LF_ERR_INVALID_ARG;
  if (splits > 32) return LF_ERR_TOO_LARGE;
  if (splits == 0)
    splits = choose_splits(a->B, a->Hkv, a->G, a->Skv, a->D, paged ? a->page_size : 0);
  // Token chunk per split: a multiple of 64 (and of the page size when that is a power of
  // two up to 64), so a split never starts in the middle of a warp's token batch.
  int chunk = round_up((a->Skv + splits - 1) / splits, 64);
  splits = (a->Skv + chunk - 1) / chunk;
  if (splits > 1) {
    const size_t need = lf_decode_workspace_bytes(a->B, a->Hkv, a->G, a->D, splits);
    if (!a->workspace || a->workspace_bytes < need) return LF_ERR_WORKSPACE;
    if (!aligned16(a->workspace)) return LF_ERR_ALIGNMENT;
  }

  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.out = static_cast<__nv_bfloat16*>(a->out);
  const int64_t units = static_cast<int64_t>(a->B) * a->Hkv * a->G;
  p.part_o = static_cast<float*>(a->workspace);
  p.part_ml = p.part_o ? p.part_o + units * splits * a->D : nullptr;
  p.block_table = a->block_table;
  p.block_table_v = a->block_table_v ? a->block_table_v : a->block_table;
  p.status = a->status;
  for (int i = 0; i < 3; ++i) {
    p.q_stride[i] = a->q_stride[i];
    p.o_stride[i] = a->o_stride[i];
    p.k_stride[i] = a->k_stride[i];
    p.v_stride[i] = a->v_stride[i];
  }
  p.bt_stride = a->bt_stride;
  p.B = a->B;
  p.Hkv = a->Hkv;
  p.Skv = a->Skv;
  p.splits = splits;
  p.chunk = chunk;
  p.page_size = paged ? a->page_size : 1;
  p.page_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == p.page_size) p.page_shift = sh;
  p.n_pages = paged ? a->n_pages : 0;
  p.scale = a->scale;
  p.mods.n = a->n_mod;
  for (int i = 0; i < LF_MAX_MODS; ++i) {
    p.mods.op[i] = i < a->n_mod ? a->mod_op[i] : 0;
    p.mods.arg[i] = i < a->n_mod ? a->mod_arg[i] : 0.f;
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  size_t smem = static_cast<size_t>(kDecodeWarps) * a->G * (a->D + 2) * sizeof(float);
  if (paged) {
    // A split's block-table slice lives in shared memory next to the K/V rings. The automatic
    // split count already keeps it small enough; an explicit count that does not is refused
    // (pass a larger `splits`, or 0).
    const size_t table_bytes = table_smem_bytes(chunk, p.page_size);
    if (table_bytes > kMaxTableBytes) return LF_ERR_TOO_LARGE;
    smem += table_bytes;
  } else if (smem > 48 * 1024) {
    return LF_ERR_TOO_LARGE;
  }

  int rc;
  if (a->D == 128)
    rc = paged ? launch_decode<128, true>(p, a->G, st, smem)
               : launch_decode<128, false>(p, a->G, st, smem);
  else
    rc = paged ? launch_decode<64, true>(p, a->G, st, smem)
               : launch_decode<64, false>(p, a->G, st, smem);
  if (rc != LF_OK) return rc;
  if (splits > 1)
    rc = lf_combine_f32(p.part_o, p.part_ml, a->out, a->B, a->Hkv, a->G, a->D, splits,
                        a->o_stride, stream);
  return rc;
}

}  // namespace lf

extern "C" {

int lf_decode_auto_splits(int32_t B, int32_t Hkv, int32_t G, int32_t Skv, int32_t D,
                          int32_t paged) {
  if (B <= 0 || Hkv <= 0 || Skv <= 0) return 1;
  int splits = lf::choose_splits(B, Hkv, G, Skv, D, paged > 0 ? paged : 0);
  const int chunk = lf::round_up((Skv + splits - 1) / splits, 64);
  return (Skv + chunk - 1) / chunk;
}

size_t lf_decode_workspace_bytes(int32_t B, int32_t Hkv, int32_t G, int32_t D, int32_t splits) {
  if (splits <= 1) return 0;
  const size_t units = static_cast<size_t>(B) * Hkv * G;
  return units * splits * (static_cast<size_t>(D) + 2) * sizeof(float);
}

int lf_decode_bf16(const LfDecodeArgs* args, void* stream) {
  return lf::decode_impl(args, stream, false);
}

int lf_decode_paged_bf16(const LfDecodeArgs* args, void* stream) {
  return lf::decode_impl(args, stream, true);
}

int lf_combine_f32(const float* part_o, const float* part_ml, void* out, int32_t B, int32_t Hkv,
                   int32_t G, int32_t D, int32_t splits, const int64_t* o_stride, void* stream) {
  if (!part_o || !part_ml || !out || !o_stride) return LF_ERR_INVALID_ARG;
  if (B <= 0 || Hkv <= 0 || G <= 0 || splits <= 0) return LF_ERR_INVALID_ARG;
  if (D != 64 && D != 128) return LF_ERR_UNSUPPORTED;
  if (splits > 32) return LF_ERR_TOO_LARGE;  // one lane per split in the combine
  const int64_t units = static_cast<int64_t>(B) * Hkv * G;
  const unsigned blocks = static_cast<unsigned>((units + 3) / 4);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 128)
    lf::combine_kernel<128><<<blocks, 128, 0, st>>>(part_o, part_ml,
                                                    static_cast<__nv_bfloat16*>(out), units, Hkv,
                                                    G, splits, o_stride[0], o_stride[1],
                                                    o_stride[2]);
  else
    lf::combine_kernel<64><<<blocks, 128, 0, st>>>(part_o, part_ml,
                                                   static_cast<__nv_bfloat16*>(out), units, Hkv,
                                                   G, splits, o_stride[0], o_stride[1],
                                                   o_stride[2]);
  return lf::check_launch("combine_kernel");
}

int lf_paged_gather_bf16(const void* pool, const int32_t* block_table, void* out, int32_t B,
                         int32_t Hkv, int32_t Skv, int32_t D, int32_t page_size, int32_t n_pages,
                         const int64_t* pool_stride, int64_t bt_stride, int32_t* status,
                         void* stream) {
  if (!pool || !block_table || !out || !pool_stride) return LF_ERR_INVALID_ARG;
  if (B <= 0 || Hkv <= 0 || Skv <= 0 || page_size <= 0 || n_pages <= 0)
    return LF_ERR_INVALID_ARG;
  if (D != 64 && D != 128) return LF_ERR_UNSUPPORTED;
  if (!lf::aligned16(pool) || !lf::aligned16(out)) return LF_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if (pool_stride[i] % 8) return LF_ERR_ALIGNMENT;
  const int64_t threads = static_cast<int64_t>(B) * Hkv * Skv * (D / 8);
  const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 128)
    lf::paged_gather_kernel<128><<<blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(pool), block_table, static_cast<__nv_bfloat16*>(out),
        B, Hkv, Skv, page_size, n_pages, pool_stride[0], pool_stride[1], pool_stride[2],
        bt_stride, status);
  else
    lf::paged_gather_kernel<64><<<blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(pool), block_table, static_cast<__nv_bfloat16*>(out),
        B, Hkv, Skv, page_size, n_pages, pool_stride[0], pool_stride[1], pool_stride[2],
        bt_stride, status);
  return lf::check_launch("paged_gather_kernel");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Decode without any allocation by the caller or the library.
//
// Some callers cannot call cudaMalloc or hand over a workspace at the point where they launch
// decode: a serving loop that has frozen its memory pool, a plugin running inside another
// runtime's callback where allocation is forbidden, or a host that only holds the input and
// output buffers it was given. For them the split-KV partials live in this fixed array, which
// is part of the library image: every GPU that loads the library holds these bytes until the
// process exits.
// ---------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[LF_STATIC_SCRATCH_BYTES];

namespace lf {

constexpr int kMaxStaticDevices = 64;
static std::mutex g_static_mutex;
static void* g_static_scratch_addr[kMaxStaticDevices] = {};

// Device address of the scratch array on the current device. `g_static_scratch` itself is only
// a host-side handle in host code, so it is translated once per device (with that device
// current) and the translated pointer is what the kernels receive.
static int static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_cuda_error(e, "cudaGetDevice");
    return LF_ERR_NO_DEVICE;
  }
  if (dev < 0 || dev >= kMaxStaticDevices) return LF_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_scratch_addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) {
      set_cuda_error(e, "cudaGetSymbolAddress(g_static_scratch)");
      cudaGetLastError();
      return LF_ERR_CUDA;
    }
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return LF_OK;
}

}  // namespace lf

extern "C" int lf_decode_bf16_static(const LfDecodeArgs* args, void* stream) {
  if (!args) return LF_ERR_INVALID_ARG;
  if (args->B <= 0 || args->Hkv <= 0 || args->G <= 0 || args->Skv <= 0)
    return LF_ERR_INVALID_ARG;
  // Resolve the split count exactly as lf_decode_bf16 will, then size the partials.
  int splits = args->splits;
  if (splits < 0) return LF_ERR_INVALID_ARG;
  if (splits == 0)
    splits = lf::choose_splits(args->B, args->Hkv, args->G, args->Skv, args->D, 0);
  const int chunk = lf::round_up((args->Skv + splits - 1) / splits, 64);
  splits = (args->Skv + chunk - 1) / chunk;
  const size_t need = lf_decode_workspace_bytes(args->B, args->Hkv, args->G, args->D, splits);
  if (need > static_cast<size_t>(LF_STATIC_SCRATCH_BYTES)) return LF_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = lf::static_scratch_address(&scratch);
  if (rc != LF_OK) return rc;
  LfDecodeArgs local = *args;
  local.splits = splits;
  local.workspace = scratch;
  local.workspace_bytes = static_cast<size_t>(LF_STATIC_SCRATCH_BYTES);
  return lf::decode_impl(&local, stream, false);
}
