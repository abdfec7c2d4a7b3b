// Prefill attention for softcap scores of bounded range, 128-key form (included by
// lf_prefill.cu, after lf_prefill_bounded.cuh whose item queue it shares).
//
// Same arithmetic as prefill_bounded_kernel (exp2 against the fixed reference 0, no running max,
// a score row split between threads with nothing to exchange but the final row sum), but the KV
// axis is walked in 128-key blocks:
//   - S_t = Q_t K^T is one set of N=128 MMAs per block (math-bound; the N=64 form of the 64-key
//     kernel is bound by the shared-memory operand reads of Q);
//   - one S buffer of 128 fp32 columns per query tile; P (bf16) overwrites the first half of the
//     32 columns each softmax thread owns;
//   - ONE issuing thread per query tile sends PV(j) and then QK^T(j+1) down the tensor pipe. The
//     pipe executes a thread's MMAs in issue order, so QK^T(j+1) may overwrite the buffer PV(j)
//     reads its P from without any completion wait in between. While the softmax warps work on
//     block j+1 of tile t, the pipe runs PV(j) and QK^T(j+1) of the other tile.
//   - the softmax warps are split by tile (eight each, two threads per score row, 64 columns per
//     thread). The two tiles run half a period apart - one in its softmax while the tensor pipe
//     works for the other - so at any time half of the warps of a scheduler compute while the
//     other half wait for scores; warps that all worked on the same block would all wait at the
//     same time.
//   - a thread takes its 64 scores as four 16-column pieces through two register buffers: the
//     load of piece c + 2 is issued as soon as piece c has been consumed, P of a piece is stored
//     right away.
// 640 threads: warps 0-7 softmax of tile 0 (row quarter = warp % 4, column half = warp / 4),
// warps 8-15 softmax of tile 1, warp 16 TMA producer and item dispatcher, warps 17/18 MMA issuers
// of tile 0/1 (the whole warp runs the loop, an elected lane issues).
// Shared memory: barrier page, 16 x 2 KB output staging, 2 Q tiles, a ring of single 128-key K or
// V tiles (4 at D=128, 8 at D=64) in consumption order K(lo), V(lo), K(lo+1), V(lo+1), ...
#pragma once

namespace lf {

constexpr int kWideK = 128;
constexpr int kWideThreads = 20 * 32;  // warp 19 only completes the register hand-over group
constexpr int kWideMaxRing = 8;

template <int D>
struct WideRingFor {
  static constexpr int value = (128 * 1024) / (kWideK * D * 2);
};

struct __align__(8) WideBarriers {
  uint64_t q_full[2];
  uint64_t q_free[2];   // [tile] last QK^T of the item has read Q_t
  uint64_t kv_full[kWideMaxRing];
  uint64_t kv_empty[kWideMaxRing];  // both MMA threads release every ring tile
  uint64_t s_full[2];   // [tile] MMA -> softmax
  uint64_t p_full[2];   // [tile] softmax -> MMA (one arrival per warp)
  uint64_t o_final[2];  // [tile] last PV of the item done
  uint64_t o_free[2];   // [tile] epilogue has read O_t (one arrival per warp)
  uint64_t l_ready[2];  // [tile] both halves of every row sum are published (one arrival per warp)
  uint64_t item_full[kItemSlots];
  uint64_t item_empty[kItemSlots];  // 2 MMA threads + 16 softmax warps have read it
  uint32_t tmem_base;
  uint32_t pad;
};

// Sixteen scores of one thread (half of its 32 columns of a 128-key block): raw scores s[] -> P
// (bf16 pairs) in pk[0..7]; row sums (over the bf16-rounded values that the PV product sees)
// into ps[]; ymax tracks max raw^2. kPath: tanh by the degree-3 polynomial, the degree-7
// polynomial, or MUFU. With kMask, columns outside [rel_lo, rel_hi] (0..15) give P = 0.
// Plain fp32 instructions: with four warps per scheduler this loop is bound by instruction issue
// (12 per pair), and the packed f32x2 forms, although fewer, take longer in their pipe (measured
// 1116 against 763 clocks per 32 x 128 scores of a scheduler).
template <int kPath, bool kMask>
__device__ __forceinline__ void wide_pass16(const PrefillParams& p, const uint32_t (&s)[16],
                                            uint32_t* pk, float (&ps)[4], float (&ymax)[2],
                                            int rel_lo, int rel_hi) {
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const float r0 = __uint_as_float(s[i]), r1 = __uint_as_float(s[i + 1]);
    const float y0 = r0 * r0, y1 = r1 * r1;
    ymax[(i >> 1) & 1] = max3(ymax[(i >> 1) & 1], y0, y1);
    float z0, z1;
    if constexpr (kPath == 0) {
      z0 = r0 * fmaf(y0, p.qc[1], p.qc[0]);
      z1 = r1 * fmaf(y1, p.qc[1], p.qc[0]);
    } else if constexpr (kPath == 1) {
      z0 = r0 * fmaf(fmaf(fmaf(y0, p.qc[3], p.qc[2]), y0, p.qc[1]), y0, p.qc[0]);
      z1 = r1 * fmaf(fmaf(fmaf(y1, p.qc[3], p.qc[2]), y1, p.qc[1]), y1, p.qc[0]);
    } else {
      z0 = tanh_approx(r0 * p.a) * p.c2;
      z1 = tanh_approx(r1 * p.a) * p.c2;
    }
    if constexpr (kMask) {
      if (i < rel_lo || i > rel_hi) z0 = -INFINITY;
      if (i + 1 < rel_lo || i + 1 > rel_hi) z1 = -INFINITY;
    }
    const uint32_t pkv = pack_bf16x2(ex2_approx(z0), ex2_approx(z1));
    pk[i >> 1] = pkv;
    if ((i >> 1) & 1) add_bf16x2_to_f32(ps[2], ps[3], pkv);
    else add_bf16x2_to_f32(ps[0], ps[1], pkv);
  }
}

template <int D>
__global__ void __launch_bounds__(kWideThreads, 1)
    prefill_wide_kernel(const __grid_constant__ CUtensorMap tmap_q,
                        const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v,
                        const __grid_constant__ CUtensorMap tmap_o, const PrefillParams p) {
  constexpr int kRing = WideRingFor<D>::value;
  constexpr int kBlocksD = D / 64;
  constexpr uint32_t kQBlockBytes = kTileQ * 128;
  constexpr uint32_t kQTileBytes = kQBlockBytes * kBlocksD;
  constexpr uint32_t kKVBlockBytes = kWideK * 128;
  constexpr uint32_t kKVTileBytes = kKVBlockBytes * kBlocksD;
  constexpr uint32_t kIdescQK = make_idesc_bf16(128, kWideK, 0);
  constexpr uint32_t kIdescPV = make_idesc_bf16(128, D, 1);
  constexpr uint32_t kColO = 256;
  constexpr int kProducerWarp = 16;
  constexpr int kMmaWarp0 = 17;

  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
  WideBarriers* bars = reinterpret_cast<WideBarriers*>(smem);
  static_assert(sizeof(WideBarriers) + 16 + kItemSlots * sizeof(ItemGeom) <= 1024, "barrier page");
  ItemGeom* item_slots =
      reinterpret_cast<ItemGeom*>(smem + ((sizeof(WideBarriers) + 15) & ~size_t(15)));
  unsigned char* sStage = smem + 1024;  // 16 x 2 KB output staging (one buffer per softmax warp)
  unsigned char* sQ = sStage + kBoundedStageBytes;
  unsigned char* sKV = sQ + 2 * kQTileBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---------------- setup ----------------
  if (warp == kMmaWarp0 && lane == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->q_full[t], 1);
      mbar_init(&bars->q_free[t], 1);
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_full[t], 8);
      mbar_init(&bars->o_final[t], 1);
      mbar_init(&bars->o_free[t], 8);
      mbar_init(&bars->l_ready[t], 8);
    }
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 2);
    }
    for (int s = 0; s < kItemSlots; ++s) {
      mbar_init(&bars->item_full[s], 1);
      mbar_init(&bars->item_empty[s], 18);
    }
    mbar_fence_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_o);
  }
  if (warp == 0) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // Next item of this role's sequence (it = -1: queue empty, or a wait ran out).
  auto next_item = [&](int seq, bool whole_warp) -> ItemGeom {
    const int slot = seq % kItemSlots;
    ItemGeom g;
    if (!mbar_wait(&bars->item_full[slot], (seq / kItemSlots) & 1)) {
      report_timeout(p.status, 20);
      g.it = -1;
      return g;
    }
    const int4* src = reinterpret_cast<const int4*>(&item_slots[slot]);
    int4 v0 = src[0], v1 = src[1], v2 = src[2];
    g.it = v0.x; g.b = v0.y; g.h = v0.z; g.hkv = v0.w;
    g.iq0 = v1.x; g.lo0 = v1.y; g.hi0 = v1.z; g.lo1 = v1.w;
    g.hi1 = v2.x; g.flags = v2.y; g.lo = v2.z; g.hi = v2.w;
    if (whole_warp) {
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->item_empty[slot]);
    } else {
      mbar_arrive(&bars->item_empty[slot]);
    }
    return g;
  };

  // The softmax warps need more registers than an even split gives them (the eight pairs of a
  // piece only overlap if each has its own temporaries): warps 16-19, one warpgroup, hand theirs
  // over. Each role changes its own allowance inside its branch.
  if (warp >= kProducerWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == kProducerWarp) {
    // ---------------- TMA producer (and item dispatcher) ----------------
    // The whole warp runs the loop; the elected lane issues the copies and publishes items.
    {
      const bool elected = elect_one_sync();
      int n = 0;             // ring position, runs across items
      int qseq[2] = {0, 0};  // items with work so far, per tile
      bool ok = true;
      auto load_tile = [&](const CUtensorMap* tma, int j, int hkv, int b) {
        if (!ok) return;
        const int stage = n % kRing;
        const uint32_t parity = ((n / kRing) & 1) ^ 1;
        ++n;
        if (!mbar_wait(&bars->kv_empty[stage], parity)) {
          report_timeout(p.status, 1);
          ok = false;
          return;
        }
        if (elected) {
          mbar_arrive_expect_tx(&bars->kv_full[stage], kKVTileBytes);
          unsigned char* dst = sKV + stage * kKVTileBytes;
#pragma unroll
          for (int kb = 0; kb < kBlocksD; ++kb)
            tma_load_4d(dst + kb * kKVBlockBytes, tma, &bars->kv_full[stage], kb * 64, j * kWideK,
                        hkv, b);
        }
        __syncwarp();
      };
      for (int seq = 0; ok; ++seq) {
        int it = 0;
        if (lane == 0) it = static_cast<int>(atomicAdd(p.ticket, 1u));
        it = __shfl_sync(0xffffffffu, it, 0);
        if (it >= p.n_items) it = -1;
        const int slot = seq % kItemSlots;
        if (!mbar_wait(&bars->item_empty[slot], ((seq / kItemSlots) & 1) ^ 1)) {
          report_timeout(p.status, 21);
          break;
        }
        ItemGeom g;
        if (it >= 0) g = decode_item(p, it, kWideK);
        else g.it = -1, g.b = g.h = g.hkv = g.iq0 = g.lo0 = g.hi0 = g.lo1 = g.hi1 = g.flags = g.lo = g.hi = 0;
        if (elected) {
          item_slots[slot] = g;
          mbar_arrive(&bars->item_full[slot]);  // release: the slot is visible to the waiters
        }
        __syncwarp();
        if (it < 0) break;
        for (int t = 0; t < 2 && ok; ++t) {
          if (!g.work(t)) continue;
          // Q_t is free once the last QK^T of the previous item with work for this tile is done.
          if (qseq[t] > 0 && !mbar_wait(&bars->q_free[t], (qseq[t] - 1) & 1)) {
            report_timeout(p.status, 22);
            ok = false;
            break;
          }
          ++qseq[t];
          if (elected) {
            mbar_arrive_expect_tx(&bars->q_full[t], kQTileBytes);
#pragma unroll
            for (int kb = 0; kb < kBlocksD; ++kb)
              tma_load_4d(sQ + t * kQTileBytes + kb * kQBlockBytes, &tmap_q, &bars->q_full[t],
                          kb * 64, (g.iq0 + t) * kTileQ, g.h, g.b);
          }
          __syncwarp();
        }
        if (g.hi > g.lo) {
          load_tile(&tmap_k, g.lo, g.hkv, g.b);
          for (int j = g.lo; j < g.hi; ++j) {
            load_tile(&tmap_v, j, g.hkv, g.b);
            if (j + 1 < g.hi) load_tile(&tmap_k, j + 1, g.hkv, g.b);
          }
        }
      }
    }
    } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // ---------------- MMA issuers: one thread per query tile ----------------
    // Both warps walk every ring tile and both release it (kv_empty counts two arrivals)
    // once the MMAs they issued from it, if any, are complete. The whole warp runs the loop
    // (every lane waits on the barriers); the elected lane alone issues MMAs and commits.
    {
      const int t = warp - kMmaWarp0;
      const bool elected = elect_one_sync();
      bool ok = true;
      constexpr uint32_t kTileUnits = kKVTileBytes >> 4;
      const uint32_t s_col = tmem_base + t * 128;
      const uint32_t o_col = tmem_base + kColO + t * 128;
      const uint64_t qdesc = make_smem_desc_sw128(smem_u32(sQ) + t * kQTileBytes, 16, 1024);
      const uint64_t kdesc0 = make_smem_desc_sw128(smem_u32(sKV), 16, 1024);
      const uint64_t vdesc0 = make_smem_desc_sw128(smem_u32(sKV), kKVBlockBytes, 1024);
      int n = 0;     // ring position, runs across items
      int gblk = 0;  // blocks of this tile so far (all items)
      int wseq = 0;  // items with work for this tile so far
      auto wait_stage = [&](int where) -> int {  // next ring tile, waited full; -1 on time-out
        const int stage = n % kRing;
        const uint32_t parity = (n / kRing) & 1;
        ++n;
        if (!mbar_wait(&bars->kv_full[stage], parity)) {
          report_timeout(p.status, where);
          ok = false;
          return -1;
        }
        return stage;
      };
      for (int seq = 0; ok; ++seq) {
        const ItemGeom g = next_item(seq, true);
        if (g.it < 0) break;
        if (g.hi <= g.lo) continue;
        const int lo = g.lo, hi = g.hi, lo_tt = g.lo_t(t), hi_tt = g.hi_t(t);
        const bool work = g.work(t);
        auto active = [&](int j) { return work && j >= lo_tt && j < hi_tt; };
        if (work) {
          if (!mbar_wait(&bars->q_full[t], wseq & 1)) {
            report_timeout(p.status, 2);
            ok = false;
            break;
          }
        }
        // S_t = Q_t K(j)^T from ring tile `stage`. The S buffer is free: the PV that read P from
        // it was issued by this thread before.
        auto issue_qk = [&](int stage, int j) {
          tc_fence_after();
          const uint64_t kd = kdesc0 + static_cast<uint64_t>(stage * kTileUnits);
          if (elected) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              mma_ss(s_col,
                     qdesc + static_cast<uint64_t>((ks / 4) * (kQBlockBytes >> 4) + (ks % 4) * 2),
                     kd + static_cast<uint64_t>((ks / 4) * (kKVBlockBytes >> 4) + (ks % 4) * 2),
                     kIdescQK, ks > 0 ? 1u : 0u);
            }
            tc_commit(&bars->s_full[t]);
            if (j == hi_tt - 1) tc_commit(&bars->q_free[t]);  // Q_t may be overwritten now
          }
          __syncwarp();
        };
        {  // K(lo)
          const int st = wait_stage(3);
          if (st < 0) break;
          if (active(lo)) issue_qk(st, lo);
          if (elected) tc_commit(&bars->kv_empty[st]);
          __syncwarp();
        }
        for (int j = lo; j < hi && ok; ++j) {
          const int sv = wait_stage(4);  // V(j)
          if (sv < 0) break;
          if (active(j)) {
            const int kt = j - lo_tt;
            const int gj = gblk + kt;
            // O_t of the previous item must have been read out before it is overwritten.
            if (kt == 0 && wseq > 0 && !mbar_wait(&bars->o_free[t], (wseq - 1) & 1)) {
              report_timeout(p.status, 14 + t);
              ok = false;
              break;
            }
            if (!mbar_wait(&bars->p_full[t], gj & 1)) {
              report_timeout(p.status, 6 + t);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint64_t vd = vdesc0 + static_cast<uint64_t>(sv * kTileUnits);
            if (elected) {
#pragma unroll
              for (int ks = 0; ks < kWideK / 16; ++ks) {
                // P of 16 keys: 8 columns; keys [64h, 64h+64) sit in the first 32 of the 64
                // columns of column half h.
                mma_ts(o_col, s_col + (ks >> 2) * 64 + (ks & 3) * 8,
                       vd + static_cast<uint64_t>(ks * (2048 >> 4)), kIdescPV,
                       (kt > 0 || ks > 0) ? 1u : 0u);
              }
              if (j == hi_tt - 1) tc_commit(&bars->o_final[t]);
            }
          }
          if (elected) tc_commit(&bars->kv_empty[sv]);
          __syncwarp();
          if (j + 1 < hi) {
            const int sk = wait_stage(5);  // K(j+1)
            if (sk < 0) break;
            if (active(j + 1)) issue_qk(sk, j + 1);
            if (elected) tc_commit(&bars->kv_empty[sk]);
            __syncwarp();
          }
        }
        if (work) {
          ++wseq;
          gblk += hi_tt - lo_tt;
        }
      }
    }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    // ---------------- softmax warps ----------------
    // Query tile t = warp / 8; inside a tile, row quarter rq = warp % 4 (the 32 tensor-memory
    // lanes this warp may touch) and column half ch = (warp / 4) % 2: the thread owns columns
    // [64 ch, 64 ch + 64) of row (32 rq + lane) of every 128-key block.
    const int t = warp >> 3;
    const int ch = (warp >> 2) & 1;
    const int rq = warp & 3;
    const int row = rq * 32 + lane;  // row inside the tile == tensor-memory lane
    const uint32_t lane_addr = static_cast<uint32_t>(rq * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + t * 128 + ch * 64;
    const uint32_t o_addr = tmem_base + lane_addr + kColO + t * 128 + ch * (D / 2);
    // Output staging of this warp; the warp that holds the other half of the same rows is
    // warp ^ 4. The two exchange their row sums through the start of each other's buffer.
    unsigned char* stage = sStage + warp * 2048;
    float* l_mine = reinterpret_cast<float*>(stage) + lane;
    float* l_partner = reinterpret_cast<float*>(sStage + (warp ^ 4) * 2048) + lane;
    // The tanh evaluation (0: degree 3, 1: degree 7, 2: MUFU) is chosen speculatively: a block
    // starts with what the warp's previous block needed, and is redone on the spot with a
    // stronger one if its own max |x| (known after the pass) asks for it.
    int path = 0;
    int gblk = 0;  // blocks of this tile so far (all items): barrier phase = gblk & 1
    int wseq = 0;  // items with work for this tile so far
    bool ok = true;
    bool store_pending = false;  // an output store of this warp may still be reading `stage`
    const int row_first = rq * 32, row_last = rq * 32 + 31;

    for (int seq = 0; ok; ++seq) {
      const ItemGeom g = next_item(seq, true);
      if (g.it < 0) break;
      const int gb = g.b, gh = g.h, iq = g.iq0 + t;
      const int grow = iq * kTileQ + row;
      if (p.dbg_ranges && g.valid(t) && row == 0 && ch == 0) {
        const int64_t idx = ((static_cast<int64_t>(gb) * p.Hq + gh) * p.n_qtiles + iq) * 2;
        p.dbg_ranges[idx] = g.lo_t(t);
        p.dbg_ranges[idx + 1] = g.hi_t(t);
      }
      if (!g.work(t)) {
        if (g.valid(t) && grow < p.Sq && ch == 0) {
          // No visible key at all for this tile: rows are NaN like the eager softmax of -inf.
          __nv_bfloat16* orow = p.out + gb * p.o_stride[0] + gh * p.o_stride[1] +
                                static_cast<int64_t>(grow) * p.o_stride[2];
          const uint4 nan4 = {0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u};
#pragma unroll
          for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = nan4;
        }
        continue;
      }
      const int lo_tt = g.lo_t(t);
      const int nblk = g.hi_t(t) - lo_tt;
      // Visible columns of a row r of this tile: [max(0, d - (window-1)), min(Skv-1, d)] with
      // d = r + diag0 for the causal kinds. c_lo and c_hi grow with the row, so the warp's first
      // and last rows decide whether a piece is fully visible or fully hidden (no votes needed).
      const int diag0 = iq * kTileQ + p.causal_offset;
      int lo_of_last = 0, lo_of_first = 0, lo_mine = 0;
      int hi_of_first = p.Skv - 1, hi_of_last = p.Skv - 1, hi_mine = p.Skv - 1;
      if (p.mask_kind != LF_MASK_NONE) {
        hi_of_first = min(p.Skv - 1, diag0 + row_first);
        hi_of_last = min(p.Skv - 1, diag0 + row_last);
        hi_mine = min(p.Skv - 1, diag0 + row);
      }
      if (p.mask_kind == LF_MASK_CAUSAL_WINDOW) {
        lo_of_first = max(0, diag0 + row_first - (p.window - 1));
        lo_of_last = max(0, diag0 + row_last - (p.window - 1));
        lo_mine = max(0, diag0 + row - (p.window - 1));
      }

      float l_run = 0.f;
#pragma unroll 1
      for (int k = 0; k < nblk; ++k) {
        const int c0 = (lo_tt + k) * kWideK + ch * 64;  // first key column of this thread
        // The time from "scores complete" to "P published" is on the critical path of the tile:
        // the wait polls, the loads go out first.
        if (!mbar_wait(&bars->s_full[t], (gblk + k) & 1)) {
          report_timeout(p.status, 8 + t);
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t sa[16], sb[16];
        tmem_ld_32x32b_x16(s_addr, sa);
        tmem_ld_32x32b_x16(s_addr + 16, sb);
        // One 16-column piece: scores in sv -> P, stored at once over columns this thread has
        // already read (piece c covers columns [16c, 16c + 16), its P goes to [8c, 8c + 8)). A
        // piece whose max |x| asks for a stronger tanh form than the warp started it with is
        // redone on the spot, from the scores still in its registers.
        auto piece = [&](uint32_t (&sv)[16], int c) {
          const int pc0 = c0 + c * 16;
          uint32_t pk[8];
          if (hi_of_last < pc0 || lo_of_first > pc0 + 15) {  // hidden for every row of the warp
#pragma unroll
            for (int i = 0; i < 8; ++i) pk[i] = 0u;
          } else {
            const bool masked = !(lo_of_last <= pc0 && hi_of_first >= pc0 + 15);
            const int rel_lo = lo_mine - pc0, rel_hi = hi_mine - pc0;
            bool again = false;
            do {
              if (again) {
                // (Read again from tensor memory - this piece's P is not stored yet and the P of
                // earlier pieces lies in lower columns - so that the scores need not stay in
                // registers through the pass.)
                tmem_ld_32x32b_x16(s_addr + c * 16, sv);
                tmem_wait_ld();
                tmem_ld_fence16(sv);
              }
              float ps[4] = {0.f, 0.f, 0.f, 0.f};
              float ymax[2] = {0.f, 0.f};
              if (path == 0) {
                if (masked) wide_pass16<0, true>(p, sv, pk, ps, ymax, rel_lo, rel_hi);
                else wide_pass16<0, false>(p, sv, pk, ps, ymax, 0, 15);
              } else if (path == 1) {
                if (masked) wide_pass16<1, true>(p, sv, pk, ps, ymax, rel_lo, rel_hi);
                else wide_pass16<1, false>(p, sv, pk, ps, ymax, 0, 15);
              } else {
                if (masked) wide_pass16<2, true>(p, sv, pk, ps, ymax, rel_lo, rel_hi);
                else wide_pass16<2, false>(p, sv, pk, ps, ymax, 0, 15);
              }
              // What this piece needed, over the whole warp (masked columns included: their raw
              // scores are ordinary finite numbers).
              const float ym = fmaxf(ymax[0], ymax[1]);
              const unsigned mine = ym > p.ylim[1] ? 2u : (ym > p.ylim[0] ? 1u : 0u);
              const int needed = static_cast<int>(__reduce_max_sync(0xffffffffu, mine));
              again = needed > path;
              path = needed;
              if (!again) l_run += (ps[0] + ps[1]) + (ps[2] + ps[3]);
            } while (again);
          }
          tmem_st8_async(s_addr + c * 8, pk);
        };
        tmem_wait_ld();
        tmem_ld_fence16(sa);
        tmem_ld_fence16(sb);
        piece(sa, 0);
        tmem_ld16_async(s_addr + 32, sa);
        piece(sb, 1);
        tmem_ld16_async(s_addr + 48, sb);
        tmem_wait_ld_async();
        tmem_ld_fence16(sa);
        tmem_ld_fence16(sb);
        piece(sa, 2);
        piece(sb, 3);
        tmem_wait_st();
        tc_fence_before();
        if (store_pending) {  // (see the epilogue) long complete by now: no real wait
          if (lane == 0) tma_store_wait_read();
          store_pending = false;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[t]);
      }
      if (!ok) break;
      gblk += nblk;

      // Row sum: each thread leaves its half in the partner's staging buffer. The partner's bulk
      // store of the previous item must have read that buffer first: the partner confirmed that
      // before its first P arrival of this item, so the completed P barrier of the item's last
      // block (eight arrivals, the partner's included) orders this write after it.
      if (!mbar_wait(&bars->p_full[t], (gblk - 1) & 1)) {
        report_timeout(p.status, 16 + t);
        ok = false;
        break;
      }
      *l_partner = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->l_ready[t]);  // (the lanes' stores are ordered first)
      if (!mbar_wait(&bars->l_ready[t], wseq & 1)) {
        report_timeout(p.status, 18 + t);
        ok = false;
        break;
      }
      l_run += *l_mine;
      __syncwarp();  // every lane has read its piece before the staging buffer is refilled
      // Epilogue: O_t / l -> bf16 -> global; each half writes D/2 of the row's columns.
      if (!mbar_wait(&bars->o_final[t], wseq & 1)) {
        report_timeout(p.status, 10 + t);
        ok = false;
        break;
      }
      ++wseq;
      tc_fence_after();
      const float inv = 1.f / l_run;
      const int row0 = iq * kTileQ + rq * 32;  // first global row of the warp
      uint32_t orr[D / 64][32];
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tmem_ld_32x32b_x32(o_addr + c * 32, orr[c]);
      tmem_wait_ld();
      // O_t is in registers: the first PV of the next item may overwrite it.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->o_free[t]);
      // 32 rows x 32 columns per bulk tensor store, staged in the 64-byte swizzle of the output
      // tensor map; rows past Sq are clipped by the hardware.
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        if (c > 0) {  // the previous box must have been read before the buffer is refilled
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t* src = &orr[c][q * 8];
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(src[0]) * inv, __uint_as_float(src[1]) * inv);
          w.y = pack_bf16x2(__uint_as_float(src[2]) * inv, __uint_as_float(src[3]) * inv);
          w.z = pack_bf16x2(__uint_as_float(src[4]) * inv, __uint_as_float(src[5]) * inv);
          w.w = pack_bf16x2(__uint_as_float(src[6]) * inv, __uint_as_float(src[7]) * inv);
          *reinterpret_cast<uint4*>(stage + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) = w;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_4d(&tmap_o, stage, ch * (D / 2) + c * 32, row0, gh, gb);
          tma_store_commit();
        }
      }
      store_pending = true;
    }
    if (lane == 0) tma_store_wait_all();  // all output stores of this warp are complete
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
