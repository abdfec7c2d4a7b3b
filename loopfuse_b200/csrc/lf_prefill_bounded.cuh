// Prefill attention for softcap scores of bounded range, persistent form (included by
// lf_prefill.cu, which holds the shared definitions and the host side).
//
// Softcap gives logit2 = c2 * tanh(a * raw) with |logit2| <= c2; when c2 <= 80, exp2(logit2) can
// be taken against the fixed reference 0 instead of a running row max. Then the blocks of a row
// are independent, O is never rescaled, and a row can be split between two threads with nothing
// to exchange but the final row sum. 672 threads:
//   warps 0-7   softmax for query tile 0: two threads per score row, 32 columns of a block each
//   warps 8-15  softmax for query tile 1
//   warp  16    TMA producer and item dispatcher
//   warps 17/18 PV issuers of tile 0 / 1, warps 19/20 QK^T issuers of tile 0 / 1 (one thread
//               each; instruction issue limits the MMA side, so the two products have their own
//               threads; the scores of block j+2 reuse the buffer that held P(j), so the QK^T
//               thread waits for the completion of PV(j))
// Tensor memory as in prefill_kernel, except that P (bf16) overwrites the first 16 columns of
// each 32-column half of its S buffer (each thread stores over its own scores).
//
// One CTA per SM walks a queue of work items (one item = two consecutive query tiles of one
// (batch, head)), taken from a ticket counter in the launch order of the non-persistent grid
// (the query-tile pairs of one head next to each other, heaviest first, so that they run at the
// same time on different SMs and share K/V through L2). Nothing drains between items:
//   - the K/V ring just continues with the next item's tiles;
//   - the S buffers of a tile keep alternating (buffer = running block count of the tile & 1), so
//     the first scores of the next item are computed while the last blocks of this one are still
//     in their softmax;
//   - Q_t of the next item is fetched as soon as the last QK^T of this item has read Q_t
//     (`q_free`), which is two blocks before the item ends;
//   - the only wait the hand-over adds is O_t: the first PV of the next item starts when the
//     epilogue has read O_t out of tensor memory (`o_free`);
//   - the output leaves through TMA bulk stores from a small staging buffer per warp, so the
//     load/store unit of the SM is not tied up by 128 scattered row segments per warp.
#pragma once

namespace lf {

constexpr int kItemSlots = 4;
constexpr int kBoundedThreads = 21 * 32;  // 16 softmax + 1 producer + 2 PV + 2 QK warps
constexpr uint32_t kBoundedStageBytes = 16 * 2048;  // 2 KB of output staging per softmax warp

struct __align__(8) BoundedBarriers {
  uint64_t q_full[2];
  uint64_t q_free[2];      // [tile] last QK^T of the item has read Q_t
  uint64_t kv_full[kMaxStages];
  uint64_t kv_empty[kMaxStages];
  uint64_t s_full[2][2];   // [tile][buffer]  MMA -> softmax
  uint64_t p_full[2][2];   // [tile][buffer]  softmax -> MMA (one arrival per warp)
  uint64_t pv_each[2][2];  // [tile][buffer]  PV of the block in that buffer done
  uint64_t o_final[2];     // [tile] last PV of the item done
  uint64_t o_free[2];      // [tile] epilogue has read O_t (one arrival per warp)
  uint64_t l_ready[2];     // [tile] both halves of every row sum are published
  uint64_t item_full[kItemSlots];   // producer -> everybody: item published
  uint64_t item_empty[kItemSlots];  // 4 MMA threads + 16 softmax warps have read it
  uint32_t tmem_base;
  uint32_t pad;
};

// Geometry of one work item: decoded once by the producer and published through shared memory
// (the divisions would otherwise be repeated by every softmax thread on the critical path).
struct ItemGeom {
  int32_t it;  // item id, -1 = queue empty
  int32_t b, h, hkv, iq0;
  int32_t lo0, hi0, lo1, hi1;  // KV block range of tile 0 / tile 1
  int32_t flags;               // bit t: tile t lies inside Sq, bit 2 + t: tile t has work
  int32_t lo, hi;              // union of the two ranges (what the K/V ring carries)
  __device__ __forceinline__ bool valid(int t) const { return (flags >> t) & 1; }
  __device__ __forceinline__ bool work(int t) const { return (flags >> (2 + t)) & 1; }
  __device__ __forceinline__ int lo_t(int t) const { return t ? lo1 : lo0; }
  __device__ __forceinline__ int hi_t(int t) const { return t ? hi1 : hi0; }
};

// `rows_q` = query rows one tile slot covers per head: 128, or 32 in the packed layout, where a
// slot holds 32 rows of each of the four query heads of one kv head (then `h` is the first of
// the four, the items run over kv heads, and iq0 counts 32-row chunks).
__device__ __forceinline__ ItemGeom decode_item(const PrefillParams& p, int it,
                                                int tile_k = kTileK, int rows_q = kTileQ) {
  ItemGeom g;
  g.it = it;
  // Heaviest query tiles of a head first. With a causal mask the lightest quarter of the pairs
  // of every head (n_deferred per head) is kept for the end of the queue: the last items that
  // the CTAs pick up are then short, so they finish close together (those pairs read only the
  // first few K/V blocks of their head again, which costs next to nothing).
  int pair, hb;
  if (it < p.main_items) {
    hb = static_cast<int>(p.div_main.div(it));
    pair = p.n_pairs - 1 - (it - hb * static_cast<int>(p.div_main.d));
  } else {
    const int r = it - p.main_items;
    hb = static_cast<int>(p.div_deferred.div(r));
    pair = p.n_deferred - 1 - (r - hb * p.n_deferred);
  }
  g.b = static_cast<int>(p.div_hq.div(hb));
  if (rows_q == kTileQ) {
    g.h = hb - g.b * p.Hq;
    g.hkv = static_cast<int>(p.div_group.div(g.h));
  } else {  // packed: div_hq divides by the number of kv heads
    g.hkv = hb - g.b * static_cast<int>(p.div_hq.d);
    g.h = g.hkv * p.group;
  }
  g.iq0 = pair * 2;
  skip_range(p.mask_kind, p.window, p.causal_offset, p.Sq, p.Skv, rows_q, tile_k, g.iq0, &g.lo0,
             &g.hi0);
  skip_range(p.mask_kind, p.window, p.causal_offset, p.Sq, p.Skv, rows_q, tile_k, g.iq0 + 1,
             &g.lo1, &g.hi1);
  const bool v0 = g.iq0 * rows_q < p.Sq, v1 = (g.iq0 + 1) * rows_q < p.Sq;
  const bool w0 = v0 && g.hi0 > g.lo0, w1 = v1 && g.hi1 > g.lo1;
  g.flags = (v0 ? 1 : 0) | (v1 ? 2 : 0) | (w0 ? 4 : 0) | (w1 ? 8 : 0);
  g.lo = 0;
  g.hi = 0;
  if (w0 && w1) {
    g.lo = min(g.lo0, g.lo1);
    g.hi = max(g.hi0, g.hi1);
  } else if (w0) {
    g.lo = g.lo0;
    g.hi = g.hi0;
  } else if (w1) {
    g.lo = g.lo1;
    g.hi = g.hi1;
  }
  return g;
}

// PACK (grouped-query attention with PACK = 2 or 4 query heads per kv head under a window
// mask; 1 = one head per tile): a tile slot holds 128 / PACK query rows of each of the PACK heads
// instead of 128 rows of one head. The keys a slot needs then span 128 / PACK + window - 1
// positions instead of 128 + window - 1 (at PACK = 4 and a window of 256: five 64-key blocks
// instead of six, and six ring stages per item instead of eight), and the heads share every K/V
// tile in shared memory, not just in L2. Tensor-memory lane quadrant q (32 rows) belongs to
// head h0 + q * PACK / 4 and holds rows (q % (4 / PACK)) * 32 .. + 32 of the slot's chunk.
template <int D, int PACK>
__global__ void __launch_bounds__(kBoundedThreads, 1)
    prefill_bounded_kernel(const __grid_constant__ CUtensorMap tmap_q,
                           const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v,
                           const __grid_constant__ CUtensorMap tmap_o, const PrefillParams p) {
  // Packed layout at D = 128 (short items: the hand-over between items is a third of the time):
  // 4 KB of output staging per warp, so that a warp's whole 32 x 64 piece of O leaves as one
  // bulk store of full 128-byte row segments and nobody waits for the store engine inside the
  // epilogue; the room comes from a K/V ring of three stages instead of four (an item has six
  // stages there). Measured on the same box: 574 -> 591 TFLOP/s on window_gqa_softcap.
  constexpr bool kBig = PACK > 1 && D == 128;
  constexpr int kStages = kBig ? 3 : StagesFor<D>::value;
  constexpr uint32_t kWarpStage = kBig ? 4096 : 2048;
  constexpr int kBlocksD = D / 64;
  static_assert(PACK == 1 || PACK == 2 || PACK == 4, "heads per tile");
  constexpr bool PACKED = PACK > 1;
  constexpr int kRowsQ = kTileQ / PACK;  // query rows of a slot per head
  constexpr uint32_t kQBlockBytes = kTileQ * 128;
  constexpr uint32_t kQTileBytes = kQBlockBytes * kBlocksD;
  constexpr uint32_t kKVBlockBytes = kTileK * 128;
  constexpr uint32_t kKVTileBytes = kKVBlockBytes * kBlocksD;
  constexpr uint32_t kIdescQK = make_idesc_bf16(128, kTileK, 0);
  constexpr uint32_t kIdescPV = make_idesc_bf16(128, D, 1);
  constexpr uint32_t kColO = 256;
  constexpr int kProducerWarp = 16;
  constexpr int kMmaWarp0 = 17;

  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
  BoundedBarriers* bars = reinterpret_cast<BoundedBarriers*>(smem);
  static_assert(sizeof(BoundedBarriers) + 16 + kItemSlots * sizeof(ItemGeom) <= 1024, "barrier page");
  static_assert(sizeof(ItemGeom) == 48, "three 16-byte pieces");
  ItemGeom* item_slots =
      reinterpret_cast<ItemGeom*>(smem + ((sizeof(BoundedBarriers) + 15) & ~size_t(15)));
  unsigned char* sStage = smem + 1024;  // 16 x 2 KB output staging (one buffer per softmax warp)
  unsigned char* sQ = sStage + 16 * kWarpStage;
  unsigned char* sKV = sQ + 2 * kQTileBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---------------- setup ----------------
  if (warp == kMmaWarp0 && lane == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->q_full[t], 1);
      mbar_init(&bars->q_free[t], 1);
      for (int bf = 0; bf < 2; ++bf) {
        mbar_init(&bars->s_full[t][bf], 1);
        mbar_init(&bars->p_full[t][bf], 8);
        mbar_init(&bars->pv_each[t][bf], 1);
      }
      mbar_init(&bars->o_final[t], 1);
      mbar_init(&bars->o_free[t], 8);
      mbar_init(&bars->l_ready[t], 256);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 4);  // every MMA thread releases every stage
    }
    for (int s = 0; s < kItemSlots; ++s) {
      mbar_init(&bars->item_full[s], 1);
      mbar_init(&bars->item_empty[s], 20);
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

  // Next item of this role's sequence (it = -1: queue empty, or a wait ran out). Every consumer
  // thread copies the slot itself; one arrival per MMA thread / softmax warp frees it.
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

  if (warp == kProducerWarp) {
    // ---------------- TMA producer (and item dispatcher) ----------------
    // The whole warp runs the loop; the elected lane issues the copies and publishes items.
    {
      const bool elected = elect_one_sync();
      int n = 0;                // ring position, runs across items
      int qseq[2] = {0, 0};     // items with work so far, per tile
      bool ok = true;
      auto load_pair = [&](const CUtensorMap* tma, int ja, int jb, int hkv, int b) {
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
          mbar_arrive_expect_tx(&bars->kv_full[stage], jb >= 0 ? 2 * kKVTileBytes : kKVTileBytes);
          unsigned char* dst = sKV + stage * (2 * kKVTileBytes);
#pragma unroll
          for (int kb = 0; kb < kBlocksD; ++kb)
            tma_load_4d(dst + kb * kKVBlockBytes, tma, &bars->kv_full[stage], kb * 64,
                        ja * kTileK, hkv, b);
          if (jb >= 0) {
#pragma unroll
            for (int kb = 0; kb < kBlocksD; ++kb)
              tma_load_4d(dst + kKVTileBytes + kb * kKVBlockBytes, &tmap_k, &bars->kv_full[stage],
                          kb * 64, jb * kTileK, hkv, b);
          }
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
        if (it >= 0) g = decode_item(p, it, kTileK, kRowsQ);
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
            if constexpr (PACKED) {  // PACK boxes of kRowsQ rows (one per head) per 64-column block
#pragma unroll
              for (int hq = 0; hq < PACK; ++hq)
#pragma unroll
                for (int kb = 0; kb < kBlocksD; ++kb)
                  tma_load_4d(sQ + t * kQTileBytes + kb * kQBlockBytes + hq * (kRowsQ * 128),
                              &tmap_q, &bars->q_full[t], kb * 64, (g.iq0 + t) * kRowsQ,
                              g.h + hq, g.b);
            } else {
#pragma unroll
              for (int kb = 0; kb < kBlocksD; ++kb)
                tma_load_4d(sQ + t * kQTileBytes + kb * kQBlockBytes, &tmap_q, &bars->q_full[t],
                            kb * 64, (g.iq0 + t) * kTileQ, g.h, g.b);
            }
          }
          __syncwarp();
        }
        if (g.hi > g.lo) {
          load_pair(&tmap_k, g.lo, g.lo + 1 < g.hi ? g.lo + 1 : -1, g.hkv, g.b);
          for (int j = g.lo; j < g.hi; ++j)
            load_pair(&tmap_v, j, j + 2 < g.hi ? j + 2 : -1, g.hkv, g.b);
        }
      }
    }
  } else if (warp >= kMmaWarp0 && warp < kMmaWarp0 + 4) {
    // ---------------- MMA issuers: a PV thread and a QK^T thread per query tile ----------
    // All four threads walk every ring stage and each releases it (kv_empty counts four
    // arrivals) once the MMAs it issued from the stage, if any, are complete. A thread must see
    // a stage full before it releases it: that keeps its arrivals one per phase.
    // The whole warp runs the loop (every lane waits on the barriers); the elected lane alone
    // issues MMAs and commits. A warp that has diverged into a single-lane branch gets far fewer
    // issue slots next to the busy softmax warps (measured: one MMA per ~150 clocks, not 64).
    {
      const int t = (warp - kMmaWarp0) & 1;
      const bool is_qk = warp - kMmaWarp0 >= 2;
      const bool elected = elect_one_sync();
      bool ok = true;
      constexpr uint32_t kStageUnits = (2 * kKVTileBytes) >> 4;  // a stage is a pair of tiles
      constexpr uint32_t kHalfUnits = kKVTileBytes >> 4;
      const uint32_t s_col = tmem_base + t * 128;
      const uint32_t o_col = tmem_base + kColO + t * 128;
      const uint64_t qdesc = make_smem_desc_sw128(smem_u32(sQ) + t * kQTileBytes, 16, 1024);
      const uint64_t kdesc0 = make_smem_desc_sw128(smem_u32(sKV), 16, 1024);
      const uint64_t vdesc0 = make_smem_desc_sw128(smem_u32(sKV), kKVBlockBytes, 1024);
      int n = 0;     // ring position, runs across items
      int gblk = 0;  // blocks of this tile so far (all items): buffer = gblk & 1
      int wseq = 0;  // items with work for this tile so far
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
      for (int seq = 0; ok; ++seq) {
        const ItemGeom g = next_item(seq, true);
        if (g.it < 0) break;
        if (g.hi <= g.lo) continue;
        const int lo = g.lo, hi = g.hi, lo_tt = g.lo_t(t), hi_tt = g.hi_t(t);
        const bool work = g.work(t);
        auto active = [&](int j) { return work && j >= lo_tt && j < hi_tt; };
        if (is_qk) {
          if (work) {
            if (!mbar_wait(&bars->q_full[t], wseq & 1)) {
              report_timeout(p.status, 2);
              ok = false;
              break;
            }
            ++wseq;
          }
          // QK^T of block j of this item (global block number gj of the tile) from K tile
          // `hf` of ring stage `stage`; its S buffer was last used by block gj - 2.
          auto issue_qk = [&](int stage, int hf, int j) -> bool {
            const int gj = gblk + (j - lo_tt);
            const int buf = gj & 1;
            if (gj >= 2 && !mbar_wait(&bars->pv_each[t][buf], ((gj - 2) >> 1) & 1)) {
              report_timeout(p.status, 12 + t);
              ok = false;
              return false;
            }
            tc_fence_after();
            const uint64_t kd =
                kdesc0 + static_cast<uint64_t>(stage * kStageUnits + hf * kHalfUnits);
            const uint32_t d = s_col + buf * 64;
            if (elected) {
#pragma unroll
              for (int ks = 0; ks < D / 16; ++ks) {
                mma_ss(d,
                       qdesc + static_cast<uint64_t>((ks / 4) * (kQBlockBytes >> 4) + (ks % 4) * 2),
                       kd + static_cast<uint64_t>((ks / 4) * (kKVBlockBytes >> 4) + (ks % 4) * 2),
                       kIdescQK, ks > 0 ? 1u : 0u);
              }
              tc_commit(&bars->s_full[t][buf]);
              if (j == hi_tt - 1) tc_commit(&bars->q_free[t]);  // Q_t may be overwritten now
            }
            __syncwarp();
            return true;
          };
          // First stage of the item: {K(lo), K(lo+1)}.
          {
            const int stage = wait_stage(3);
            if (stage < 0) break;
            tc_fence_after();
            if (active(lo) && !issue_qk(stage, 0, lo)) break;
            if (lo + 1 < hi && active(lo + 1) && !issue_qk(stage, 1, lo + 1)) break;
            if (elected) tc_commit(&bars->kv_empty[stage]);
            __syncwarp();
          }
          for (int j = lo; j < hi && ok; ++j) {
            const int st = wait_stage(4);  // {V(j), K(j+2)}
            if (st < 0) break;
            if (j + 2 < hi && active(j + 2)) {
              tc_fence_after();
              if (!issue_qk(st, 1, j + 2)) break;
            }
            if (elected) tc_commit(&bars->kv_empty[st]);
            __syncwarp();
          }
        } else {
          {  // the first stage of an item holds K tiles only
            const int st = wait_stage(5);
            if (st < 0) break;
            if (elected) tc_commit(&bars->kv_empty[st]);
            __syncwarp();
          }
          for (int j = lo; j < hi && ok; ++j) {
            const int st = wait_stage(5);  // {V(j), K(j+2)}
            if (st < 0) break;
            if (active(j)) {
              const int kt = j - lo_tt;
              const int gj = gblk + kt;
              // O_t of the previous item must have been read out before it is overwritten.
              if (kt == 0 && wseq > 0 && !mbar_wait(&bars->o_free[t], (wseq - 1) & 1)) {
                report_timeout(p.status, 14 + t);
                ok = false;
                break;
              }
              if (!mbar_wait(&bars->p_full[t][gj & 1], (gj >> 1) & 1)) {
                report_timeout(p.status, 6 + t);
                ok = false;
                break;
              }
              tc_fence_after();
              const uint64_t vd = vdesc0 + static_cast<uint64_t>(st * kStageUnits);
              const uint32_t a = s_col + (gj & 1) * 64;
              if (elected) {
#pragma unroll
                for (int ks = 0; ks < kTileK / 16; ++ks) {
                  // P columns of 16 keys: 16 columns at the start of each 32-column half of S.
                  mma_ts(o_col, a + (ks >> 1) * 32 + (ks & 1) * 8,
                         vd + static_cast<uint64_t>(ks * (2048 >> 4)), kIdescPV,
                         (kt > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(&bars->pv_each[t][gj & 1]);
                if (j == hi_tt - 1) tc_commit(&bars->o_final[t]);
              }
            }
            if (elected) tc_commit(&bars->kv_empty[st]);
            __syncwarp();
          }
          if (work) ++wseq;
        }
        if (work) gblk += hi_tt - lo_tt;
      }
    }
  } else {
    // ---------------- softmax warps ----------------
    // Query tile t = warpgroup / 2; inside a tile, warpgroup `half` takes columns
    // [32*half, 32*half + 32) of every 64-key block, one thread per (row, half). With the fixed
    // reference there is no running max, no rescale of O and nothing to exchange between the
    // two threads of a row until the final row sum.
    const int wg = warp >> 2;
    const int t = wg >> 1;
    const int half = wg & 1;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // row inside the tile == tensor-memory lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_base = tmem_base + lane_addr + t * 128 + half * 32;
    const uint32_t o_addr = tmem_base + lane_addr + kColO + t * 128;
    // Output staging of this warp; the warp that holds the other half of the same rows is
    // warp ^ 4. The two exchange their row sums through the start of each other's buffer.
    unsigned char* stage = sStage + warp * kWarpStage;
    float* l_mine = reinterpret_cast<float*>(stage) + lane;
    float* l_partner = reinterpret_cast<float*>(sStage + (warp ^ 4) * kWarpStage) + lane;
    // tanh(x) = x*(1 + y*(-1/3 + y*(2/15 + y*(-17/315)))), y = x^2, x = a*raw. The powers of a and
    // the output factor c2 are folded into the coefficients p.qc[] on the host, so the polynomial
    // runs on raw^2 and gives logit2 = raw * q(raw^2) directly; p.ylim[] are the limits of the two
    // polynomials as bounds on raw^2.
    // The tanh evaluation (0: degree 3, 1: degree 7, 2: MUFU) is chosen speculatively: a block
    // starts with what the warp's previous block needed, and is redone on the spot with a
    // stronger one if its own max |x| (known after the pass) asks for it.
    int path = 0;
    int gblk = 0;  // blocks of this tile so far (all items): buffer = gblk & 1
    int wseq = 0;  // items with work for this tile so far
    bool ok = true;
    bool store_pending = false;  // an output store of this warp may still be reading `stage`
    for (int seq = 0; ok; ++seq) {
      const ItemGeom g = next_item(seq, true);
      if (g.it < 0) break;
      // row of this thread inside its head's chunk, and that head
      const int crow = (quarter % (4 / PACK)) * 32 + lane;
      const int grow = (g.iq0 + t) * kRowsQ + crow;
      const int head = g.h + quarter * PACK / 4;
      if (p.dbg_ranges && g.valid(t) && crow == 0 && half == 0) {
        const int64_t idx =
            ((static_cast<int64_t>(g.b) * p.Hq + head) * p.n_qtiles + (g.iq0 + t)) * 2;
        p.dbg_ranges[idx] = g.lo_t(t);
        p.dbg_ranges[idx + 1] = g.hi_t(t);
      }
      if (!g.work(t)) {
        if (g.valid(t) && grow < p.Sq && half == 0) {
          // No visible key at all for this tile: softmax of an all -inf row is NaN in the
          // eager computation, so the rows are written as NaN.
          __nv_bfloat16* orow = p.out + g.b * p.o_stride[0] + head * p.o_stride[1] +
                                static_cast<int64_t>(grow) * p.o_stride[2];
          const uint4 nan4 = {0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u};
#pragma unroll
          for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = nan4;
        }
        continue;
      }
      // Visible column interval of this row: [c_lo, c_hi].
      int c_hi = p.Skv - 1;
      int c_lo = 0;
      if (p.mask_kind != LF_MASK_NONE) c_hi = min(c_hi, grow + p.causal_offset);
      if (p.mask_kind == LF_MASK_CAUSAL_WINDOW)
        c_lo = max(0, grow + p.causal_offset - (p.window - 1));

      float l_run = 0.f;
      const int lo_tt = g.lo_t(t);
      const int nblk = g.hi_t(t) - lo_tt;
      for (int k = 0; k < nblk; ++k) {
        const int c0 = (lo_tt + k) * kTileK + half * 32;  // first key column of this thread
        const int gk = gblk + k;
        const int buf = gk & 1;
        const uint32_t s_addr = s_base + buf * 64;
        if (!mbar_wait(&bars->s_full[t][buf], (gk >> 1) & 1)) {
          report_timeout(p.status, 8 + t);
          ok = false;
          break;
        }
        tc_fence_after();
        const int rel_lo = c_lo - c0;  // visible columns of this thread's 32: [rel_lo, rel_hi]
        const int rel_hi = c_hi - c0;
        // Warp-uniform decisions (the 32 x 32 piece of the block that this warp owns is fully
        // visible, crossed by a mask edge, or fully hidden), so that a warp never runs both
        // forms of the pass and a hidden piece costs nothing.
        const bool masked = __any_sync(0xffffffffu, rel_lo > 0 || rel_hi < 31);
        const bool hidden = __all_sync(0xffffffffu, rel_lo > 31 || rel_hi < 0);

        uint32_t pk[16];
        float block_sum = 0.f;
        if (hidden) {
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = 0u;
        }
        while (!hidden) {
          // (Read again from tensor memory when a block is redone: P is stored only at the end.)
          uint32_t sr[32];
          tmem_ld_32x32b_x32(s_addr, sr);
          tmem_wait_ld();
          float psum[4] = {0.f, 0.f, 0.f, 0.f};
          float ymax0 = 0.f, ymax1 = 0.f;
          // Plain fp32 instructions: this loop is bound by instruction issue (12 per pair), and
          // the packed f32x2 forms, although fewer, take longer in their pipe (measured 1116
          // against 763 clocks per 32 x 128 scores of a scheduler).
          auto body = [&](auto path_tag, bool apply_mask) {
            constexpr int kPath = decltype(path_tag)::value;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float r0 = __uint_as_float(sr[i]), r1 = __uint_as_float(sr[i + 1]);
              const float y0 = r0 * r0, y1 = r1 * r1;
              if ((i >> 1) & 1) ymax1 = max3(ymax1, y0, y1); else ymax0 = max3(ymax0, y0, y1);
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
              if (apply_mask) {
                if (i < rel_lo || i > rel_hi) z0 = -INFINITY;
                if (i + 1 < rel_lo || i + 1 > rel_hi) z1 = -INFINITY;
              }
              // The row sum is taken over the bf16-rounded values that the PV product sees, so
              // that numerator and denominator carry the same rounding (the largest P of a row
              // is not exactly 1 as it would be with a running max). The mixed-precision add
              // reads the bf16 halves directly.
              const uint32_t pkv = pack_bf16x2(ex2_approx(z0), ex2_approx(z1));
              pk[i >> 1] = pkv;
              if ((i >> 1) & 1) add_bf16x2_to_f32(psum[2], psum[3], pkv);
              else add_bf16x2_to_f32(psum[0], psum[1], pkv);
            }
          };
          if (path == 0) {
            if (masked) body(std::integral_constant<int, 0>{}, true);
            else body(std::integral_constant<int, 0>{}, false);
          } else if (path == 1) {
            if (masked) body(std::integral_constant<int, 1>{}, true);
            else body(std::integral_constant<int, 1>{}, false);
          } else {
            if (masked) body(std::integral_constant<int, 2>{}, true);
            else body(std::integral_constant<int, 2>{}, false);
          }
          block_sum = (psum[0] + psum[1]) + (psum[2] + psum[3]);
          // What this block needed, over the whole warp (masked columns included: their raw
          // scores are ordinary finite numbers).
          const float ymax = fmaxf(ymax0, ymax1);
          const unsigned mine = ymax > p.ylim[1] ? 2u : (ymax > p.ylim[0] ? 1u : 0u);
          const int needed = static_cast<int>(__reduce_max_sync(0xffffffffu, mine));
          const bool redo = needed > path;
          path = needed;
          if (!redo) break;
        }
        l_run += block_sum;
        // P (bf16, two per column) goes on top of the first 16 of this thread's S columns.
        tmem_st_32x32b_x16(s_addr, pk);
        tmem_wait_st();
        tc_fence_before();
        if (store_pending) {  // (see the epilogue) long complete by now: no real wait
          if (lane == 0) tma_store_wait_read();
          store_pending = false;
        }
        // One arrival per warp (256 arrivals on one barrier word would serialise).
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[t][buf]);
      }
      if (!ok) break;
      gblk += nblk;

      // Row sum: each thread leaves its half in the partner's staging buffer. The partner's bulk
      // store of the previous item must have read that buffer first: the partner confirmed that
      // before its first P arrival of this item, so the completed P barrier of the item's last
      // block (eight arrivals, the partner's included) orders this write after it. (Without this
      // wait an item of one or two blocks gave no such ordering.)
      if (!mbar_wait(&bars->p_full[t][(gblk - 1) & 1], ((gblk - 1) >> 1) & 1)) {
        report_timeout(p.status, 16 + t);
        ok = false;
        break;
      }
      *l_partner = l_run;
      mbar_arrive(&bars->l_ready[t]);
      if (!mbar_wait(&bars->l_ready[t], wseq & 1)) {
        report_timeout(p.status, 18 + t);
        ok = false;
        break;
      }
      l_run += *l_mine;
      // Epilogue: O_t / l -> bf16 -> global; each half writes D/2 of the row's columns.
      if (!mbar_wait(&bars->o_final[t], wseq & 1)) {
        report_timeout(p.status, 10 + t);
        ok = false;
        break;
      }
      ++wseq;
      tc_fence_after();
      const float inv = 1.f / l_run;
      // first global row of the warp
      const int row0 = (g.iq0 + t) * kRowsQ + (quarter % (4 / PACK)) * 32;
      // The warp's 32 rows x 32 columns go to its staging buffer in the 64-byte swizzle of the
      // output tensor map (16-byte piece q of row r at position q ^ ((r >> 1) & 3), conflict
      // free), and one bulk tensor store moves them to global memory; rows past Sq are clipped
      // by the hardware. The store engine, not the load/store unit of the SM, writes the
      // 32 x 64-byte row segments.
      // Long items (kLoadAll): all of the warp's O columns are loaded first, so that O_t is
      // released as early as possible. Short items (the packed layout): one 32-column box at a
      // time, so that the tensor-memory load of the next box runs while the store engine reads
      // the previous one out of the staging buffer (measured: +1.5 % there, -0.5 % on long items).
      constexpr bool kLoadAll = !PACKED || kBig;
      uint32_t orr[D / 64][32];
      if constexpr (kLoadAll) {
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tmem_ld_32x32b_x32(o_addr + half * (D / 2) + c * 32, orr[c]);
        tmem_wait_ld();
        // O_t is in registers: the first PV of the next item may overwrite it.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->o_free[t]);
      }
      if constexpr (kBig) {
        // 128-byte rows: 16-byte piece q of row r at position q ^ (r & 7) (the 128-byte swizzle
        // of the 64-column output map), one store for the warp's whole piece.
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint32_t* src = &orr[q >> 2][(q & 3) * 8];
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(src[0]) * inv, __uint_as_float(src[1]) * inv);
          w.y = pack_bf16x2(__uint_as_float(src[2]) * inv, __uint_as_float(src[3]) * inv);
          w.z = pack_bf16x2(__uint_as_float(src[4]) * inv, __uint_as_float(src[5]) * inv);
          w.w = pack_bf16x2(__uint_as_float(src[6]) * inv, __uint_as_float(src[7]) * inv);
          *reinterpret_cast<uint4*>(stage + lane * 128 + ((q ^ (lane & 7)) << 4)) = w;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_4d(&tmap_o, stage, half * 64, row0, head, g.b);
          tma_store_commit();
        }
      } else
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        if constexpr (!kLoadAll) {
          tmem_ld_32x32b_x32(o_addr + half * (D / 2) + c * 32, orr[c]);
          tmem_wait_ld();
          if (c == D / 64 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->o_free[t]);
          }
        }
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
          tma_store_4d(&tmap_o, stage, half * (D / 2) + c * 32, row0, head, g.b);
          tma_store_commit();
        }
      }
      // The buffer is written again (by the partner, with its row sum) at the end of the next
      // item; this warp confirms that the store has read it before its first P of that item.
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
