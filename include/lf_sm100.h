/*
 * lf_sm100.h - C ABI of liblf_sm100.so: hand-written sm_100a (B200) kernels for the fused
 * attention hot path that the loopfuse compiler generates.
 *
 * Every entry point takes plain device pointers, element strides and sizes; nothing in
 * the signatures depends on PyTorch. Pointers are borrowed (never freed by the library).
 * All launches are asynchronous on the CUDA stream passed in (a cudaStream_t carried as
 * void*; NULL = the legacy default stream). Return value: LF_OK, or a negative LfStatus
 * for argument / launch errors detected on the host. Device-side problems (a bounded wait
 * that ran out, a page id outside the pool) are written to the optional `status` device
 * word as a positive code; the kernels never trap.
 *
 * Reference interface each entry replaces (paths inside tomatillos/loopfuse):
 *   lf_prefill_bf16        the generated launcher + kernel for prefill graphs:
 *                          loopfuse/codegen.py:215-298 (launch_kernel_0), :454-998 (body);
 *                          called from loopfuse/torch_backend/interface.py:640-644.
 *   lf_decode_bf16         same generator, M==1 special case loopfuse/codegen.py:661-663.
 *   lf_decode_paged_bf16   same, with the two-level paged load loopfuse/codegen.py:738-872
 *                          (op: loopfuse/torch_backend/__init__.py:46-63).
 *   lf_combine_f32         no reference counterpart as a separate kernel: the reference runs
 *                          the whole KV loop in one program (README.md:117 lists split-k as
 *                          missing); this merges split-KV partial results.
 *   lf_paged_gather_bf16   the eager gather buffer[block_table]
 *                          (loopfuse/torch_backend/__init__.py:46-56), used to check page
 *                          indexing bit for bit.
 *   lf_skip_range          the loop-range rewrite of the sparsity pass,
 *                          loopfuse/compiler/passes/skip_loop_iterations.py:343-376.
 *   lf_kv_append_bf16      the write side of the paged cache the two-level load reads: the
 *                          cache / block-table layout of tests/benchmark.py:308-319 and the
 *                          index rule of loopfuse/torch_backend/__init__.py:46-63
 *                          (out = buffer[block_table]), used as a store address. The reference
 *                          fills its caches on the host with torch.randn.
 */
#ifndef LF_SM100_H_
#define LF_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LF_ABI_VERSION 5

typedef enum {
  LF_OK = 0,
  LF_ERR_INVALID_ARG = -1,   /* NULL pointer, bad size, unsupported head dim ...            */
  LF_ERR_UNSUPPORTED = -2,   /* valid request that this build has no kernel for             */
  LF_ERR_ALIGNMENT = -3,     /* pointer / stride not aligned as the kernels require         */
  LF_ERR_WORKSPACE = -4,     /* split-KV workspace missing or too small                     */
  LF_ERR_CUDA = -5,          /* a CUDA runtime / driver call failed (see lf_last_cuda_error) */
  LF_ERR_NO_DEVICE = -6,     /* no sm_100 device is current                                 */
  LF_ERR_TOO_LARGE = -7      /* size beyond a fixed limit of the entry point                */
} LfStatus;

/* Codes the kernels write to the `status` device word (0 = nothing happened). */
#define LF_DEV_OK 0
#define LF_DEV_TIMEOUT 1        /* a bounded mbarrier wait gave up; low bits say which      */
#define LF_DEV_BAD_PAGE 2       /* block_table entry outside [0, n_pages)                   */
#define LF_DEV_BOUNDS 3         /* debug-bounds build only: an index left its range; bits 8..
                                   say where. The access was skipped or clamped.            */

/* Mask kinds (what the capture layer deduces from loopfuse::causal_mask / sliding_mask). */
#define LF_MASK_NONE 0
#define LF_MASK_CAUSAL 1          /* keep j <= i + causal_offset                             */
#define LF_MASK_CAUSAL_WINDOW 2   /* keep i + off - (window-1) <= j <= i + off               */

/* Score-mod opcodes: applied in order to s = scale * (q . k) before the mask. */
#define LF_MOD_MUL 1     /* s *= arg   */
#define LF_MOD_ADD 2     /* s += arg   */
#define LF_MOD_TANH 3
#define LF_MOD_EXP 4
#define LF_MOD_EXP2 5
#define LF_MOD_SIN 6
#define LF_MOD_COS 7
#define LF_MOD_RELU 8
#define LF_MOD_SQUARE 9
#define LF_MOD_DIV 10    /* s /= arg   */
#define LF_MAX_MODS 8

/* Prefill tile shapes of the sm_100a kernels; skip ranges are defined on them. Query tiles are
 * always 128 rows; KV tiles are 64 keys, or 128 keys in the wide bounded-softcap kernel (see
 * lf_prefill_kv_tile). */
#define LF_PREFILL_TILE_Q 128
#define LF_PREFILL_TILE_K 64
#define LF_PREFILL_TILE_K_WIDE 128

typedef struct {
  const void* q;      /* bf16 [B, Hq,  Sq,  D], innermost stride 1 */
  const void* k;      /* bf16 [B, Hkv, Skv, D] */
  const void* v;      /* bf16 [B, Hkv, Skv, D] */
  void* out;          /* bf16 [B, Hq,  Sq,  D] */
  int32_t B, Hq, Hkv, Sq, Skv, D;   /* D in {64, 128}; Hq % Hkv == 0 */
  int64_t q_stride[3];  /* element strides of dims (b, h, s) */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  float scale;          /* first multiplier of q.k (D^-0.5 in the usual case) */
  int32_t n_mod;        /* 0..LF_MAX_MODS */
  int32_t mod_op[LF_MAX_MODS];
  float mod_arg[LF_MAX_MODS];
  int32_t mask_kind;    /* LF_MASK_* */
  int32_t window;       /* for LF_MASK_CAUSAL_WINDOW */
  int32_t causal_offset;/* 0 for square scores */
  int32_t* status;      /* optional device word */
  int32_t* dbg_ranges;  /* optional device int32 [B*Hq*ceil(Sq/128)*2]: the (lo,hi) range of
                           KV tiles (of lf_prefill_kv_tile(args) keys) each q-tile actually
                           iterated (bit-exact check against lf_skip_range) */
  int32_t kv_tile;      /* 0 = the library picks; 64 or 128 pins the KV tile of the kernel
                           (128 exists only for the bounded-softcap kernel) */
  /* Paged K and / or V (NULL tables = dense operands). With k_block_table, `k` is a pool
   * [n_pages, page_size, Hkv, D] and k_stride its element strides of (page, slot, kv head);
   * key t of sequence b is pool[k_block_table[b, t / page_size], t % page_size, kv head, :]
   * for t < Skv. Likewise v_block_table / v / v_stride. The gather is fused into the tile load
   * of the kernel (the reference's two-level load, loopfuse/codegen.py:738-872); an entry
   * outside [0, n_pages) is reported as LF_DEV_BAD_PAGE in `status` and read as page 0. */
  const int32_t* k_block_table; /* int32 [B, >= ceil(Skv / page_size)] */
  const int32_t* v_block_table;
  int64_t bt_stride;            /* elements between rows of the tables */
  int32_t page_size;
  int32_t n_pages;
  int32_t sm_margin;    /* persistent kernels only: leave this many SMs without a CTA, for
                           kernels that must run at the same time (a collective on another
                           stream cannot start while one CTA per SM is resident); 0 = use all */
  /* Additive score bias (NULL = none): bf16 [B, Hq, Sq, Skv], innermost stride 1, 16-byte
   * aligned rows; bias_stride = element strides of (b, h, row). It is added to the score after
   * the first `bias_pos` ops of the mod chain (0 <= bias_pos <= n_mod) and before the mask:
   *     s = mod[bias_pos .. n_mod)( mod[0 .. bias_pos)(scale * q.k) + bias[b, h, i, j] )
   * - the `QK * c + scores_bias` form of the reference's modified-attention test
   * (tests/test_accuracy.py:176-194), read tile by tile inside the kernel. Dense K/V only. */
  const void* score_bias;
  int64_t bias_stride[3];
  int32_t bias_pos;
  /* Second score product (NULL = none): scores = scale * (q k^T + q_pe k_pe^T), the two-matmul
   * form of the reference's MLA test (tests/test_attention.py:126-151). q_pe bf16 [B, Hq, Sq,
   * D_pe], k_pe bf16 [B, Hkv, Skv, D_pe], D_pe in {8, 16, ..., 64}, innermost stride 1, rows
   * 16-byte aligned. Dense K/V, no score bias, and a mod chain of constant multipliers only
   * (anything else is LF_ERR_UNSUPPORTED). */
  const void* q_pe;
  const void* k_pe;
  int64_t qpe_stride[3];
  int64_t kpe_stride[3];
  int32_t D_pe;
} LfPrefillArgs;

typedef struct {
  const void* q;        /* bf16 [B, Hkv, G, D]: the G query heads that share a kv head */
  const void* k;        /* dense: bf16 [B, Hkv, Skv, D]. paged: pool [n_pages, page_size, Hkv, D] */
  const void* v;
  void* out;            /* bf16 [B, Hkv, G, D] */
  int32_t B, Hkv, G, Skv, D;   /* D in {64, 128}; G in {1, 2, 4, 8} */
  int64_t q_stride[3];  /* (b, hkv, g) */
  int64_t o_stride[3];
  int64_t k_stride[3];  /* dense: (b, hkv, s). paged: (page, slot, hkv) */
  int64_t v_stride[3];
  float scale;
  int32_t n_mod;
  int32_t mod_op[LF_MAX_MODS];
  float mod_arg[LF_MAX_MODS];
  /* paged only */
  const int32_t* block_table;   /* int32 [B, ceil(Skv/page_size)]: pages of K (and of V) */
  const int32_t* block_table_v; /* pages of V when they differ from K's; NULL = same table */
  int64_t bt_stride;            /* elements between rows of block_table */
  int32_t page_size;
  int32_t n_pages;
  /* split-KV */
  int32_t splits;               /* 1..32; 0 = let the library choose */
  void* workspace;              /* device, >= lf_decode_workspace_bytes(...) when splits != 1 */
  size_t workspace_bytes;
  int32_t* status;              /* optional device word */
} LfDecodeArgs;

typedef struct {
  const void* k_new;    /* bf16 [B, Hkv, T, D]: T new key rows per sequence, innermost stride 1 */
  const void* v_new;    /* bf16 [B, Hkv, T, D] */
  void* k_pool;         /* bf16 [n_pages, page_size, Hkv, D] (page_size 1: [n_pages, Hkv, D]) */
  void* v_pool;
  const int32_t* block_table;   /* int32 [B, bt_blocks]: pages of K (and of V) */
  const int32_t* block_table_v; /* pages of V when they differ from K's; NULL = same table */
  const int32_t* seq_pos;       /* device int32 [B]: logical position of each sequence's first
                                   new token; NULL = start_pos for every sequence */
  int32_t start_pos;
  int32_t B, Hkv, T, D;         /* D in {64, 128} */
  int64_t kn_stride[3];         /* element strides of k_new dims (b, hkv, t) */
  int64_t vn_stride[3];
  int64_t kp_stride[3];         /* element strides of k_pool dims (page, slot, hkv) */
  int64_t vp_stride[3];
  int64_t bt_stride;            /* elements between rows of block_table */
  int32_t bt_blocks;            /* entries per row of block_table */
  int32_t page_size;
  int32_t n_pages;
  int32_t* status;              /* optional device word */
} LfKvAppendArgs;

typedef struct {
  int32_t abi_version;
  int32_t device;         /* current CUDA device ordinal */
  int32_t cc_major, cc_minor;
  int32_t sm_count;
  int32_t max_smem_optin; /* bytes */
  int64_t total_mem;
} LfDeviceInfo;

/* Fill *info for the current device. */
int lf_query(LfDeviceInfo* info);

const char* lf_strerror(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* lf_last_cuda_error(void);

/* Prefill attention: out = softmax(mask(mod(scale * q k^T))) v, online softmax, tcgen05 MMA.
 * A score-mod chain of the softcap form (MUL|DIV)* TANH (MUL|DIV)* with cap * log2(e) <= 80 (and
 * Skv <= 2^22) runs a persistent kernel that takes exp2 against the fixed reference 0 instead
 * of a running row max: P lies in [2^-80, 2^80], row sums and outputs are accumulated in fp32.
 * That is exact softmax arithmetic (same result within the bf16 tolerance) as long as
 * Skv * max|v| stays below about 2^46 (e.g. |v| < 2^24 at the largest Skv); beyond that the fp32
 * accumulators can overflow where the running-max form would not. Every other chain uses the
 * running-max kernel. The persistent kernel keeps its work-queue counters in the library image
 * (256 slots taken round-robin and zeroed in stream order): more than 256 such launches in
 * flight at once on one device could share a counter. A launch recorded into a CUDA graph keeps
 * the slot it was given at capture time for as long as the graph lives, while eager launches
 * keep cycling through the slots: keep replays of such a graph and eager launches of the
 * persistent kernel on one stream (or ordered), or every 256th eager launch could share the
 * replay's counter and lose work items. The first call of each kernel variant (head dim,
 * score-function mode) on a host thread sets kernel attributes and looks up symbol addresses:
 * make it outside stream capture, from the thread that will capture. */
int lf_prefill_bf16(const LfPrefillArgs* args, void* stream);
/* KV tile size (64 or 128 keys) of the kernel lf_prefill_bf16 would run for these arguments, or
 * a negative LfStatus; launches nothing. Skip ranges and `dbg_ranges` are in units of it.
 * Replaces the tile sizes the reference autotunes per kernel (loopfuse/codegen.py:360-393). */
int lf_prefill_kv_tile(const LfPrefillArgs* args);
/* Query rows per head that one tile of that kernel covers: LF_PREFILL_TILE_Q, or 128 / g when
 * the library packs the g = Hq / Hkv query heads of a kv head into one tile (grouped-query
 * attention with g in {2, 4} under a window mask and a softcap chain). `dbg_ranges` then holds
 * one (lo, hi) per (batch, query head, chunk of that many rows): int32 [B * Hq * ceil(Sq /
 * q_tile) * 2]. Negative LfStatus on error; launches nothing. */
int lf_prefill_q_tile(const LfPrefillArgs* args);
/* Hit / miss counters of the library's cache of encoded tensor maps (keyed by address, shape,
 * strides and box; the per-call host work the reference's launcher repeats on every call,
 * loopfuse/codegen.py:215-298). Either pointer may be NULL. */
void lf_tile_map_cache_stats(uint64_t* hits, uint64_t* misses);

/* KV-tile range [lo, hi) that q-tile `iq` must visit; the same integers the kernel uses. */
void lf_skip_range(int32_t mask_kind, int32_t window, int32_t causal_offset, int32_t Sq,
                   int32_t Skv, int32_t tile_q, int32_t tile_k, int32_t iq, int32_t* lo,
                   int32_t* hi);

/* Decode attention (Sq == 1 per head, G grouped heads per kv head), split over KV. */
int lf_decode_bf16(const LfDecodeArgs* args, void* stream);
int lf_decode_paged_bf16(const LfDecodeArgs* args, void* stream);
/* Split count the library picks for splits == 0, and the workspace it then needs. `page_size`
 * is 0 for a dense cache, else the tokens per page of the paged cache (a split's slice of the
 * block table is staged in shared memory; with small pages and a long context the library splits
 * further until the slice fits, and an explicit split count that leaves it too large is refused
 * with LF_ERR_TOO_LARGE). */
int lf_decode_auto_splits(int32_t B, int32_t Hkv, int32_t G, int32_t Skv, int32_t D,
                          int32_t page_size);
size_t lf_decode_workspace_bytes(int32_t B, int32_t Hkv, int32_t G, int32_t D, int32_t splits);

/* Decode for callers that cannot allocate. No counterpart in the reference (it has neither
 * split-KV nor a workspace). Same arguments and result as lf_decode_bf16, except that
 * `workspace` / `workspace_bytes` are ignored: the split-KV partials go to a fixed array of
 * LF_STATIC_SCRATCH_BYTES that is part of the library image (each GPU that loads the library
 * holds it until the process exits). Meant for hosts that may not call cudaMalloc at launch
 * time - a serving loop with a frozen memory pool, a plugin called from inside another
 * runtime - and only own their input and output buffers.
 *   - Nothing is allocated or freed, by this call or by anything it calls.
 *   - A problem whose partials (lf_decode_workspace_bytes for the resolved split count) exceed
 *     LF_STATIC_SCRATCH_BYTES is refused with LF_ERR_TOO_LARGE; pass a smaller `splits`.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array. Its old contents never matter (every partial
 *     that is read was written by the same call), but two calls that run on the GPU at the
 *     same time - different streams, or different threads - overwrite each other's partials:
 *     keep calls on one device ordered. */
#define LF_STATIC_SCRATCH_BYTES (8u << 20)
int lf_decode_bf16_static(const LfDecodeArgs* args, void* stream);

/* Merge split-KV partials: part_o fp32 [units, splits, D], part_ml fp32 [units, splits, 2]
 * (running max in log2 domain, sum) -> out bf16 rows; out row u lives at
 * out + (u / G / Hkv) * o_stride[0] + ((u / G) % Hkv) * o_stride[1] + (u % G) * o_stride[2]. */
int lf_combine_f32(const float* part_o, const float* part_ml, void* out, int32_t B, int32_t Hkv,
                   int32_t G, int32_t D, int32_t splits, const int64_t* o_stride, void* stream);

/* Gather only: out[b, h, t, :] = pool[block_table[b, t / page_size], t % page_size, h, :]. */
int lf_paged_gather_bf16(const void* pool, const int32_t* block_table, void* out, int32_t B,
                         int32_t Hkv, int32_t Skv, int32_t D, int32_t page_size, int32_t n_pages,
                         const int64_t* pool_stride, int64_t bt_stride, int32_t* status,
                         void* stream);

/* Self-test of the bounded device-side waits (no counterpart in the reference, whose kernels
 * have no cross-warp waits): a one-thread kernel waits at most `limit_cycles` SM clocks on an
 * mbarrier that nobody arrives on, then records LF_DEV_TIMEOUT | (99 << 8) in `status` (device
 * word, required) and the clocks it really waited in `waited_cycles` (device int64, optional),
 * and returns. Shows on a live GPU what every kernel of the library does when a wait does not
 * complete: give up, report, terminate normally. limit_cycles in (0, 2e9]. */
int lf_selftest_wait_timeout(int64_t limit_cycles, int32_t* status, int64_t* waited_cycles,
                             void* stream);

/* Append to a paged KV cache: new token i of sequence b (logical position pos = seq_pos[b] + i,
 * or start_pos + i) is written to
 *     pool[block_table[b, pos / page_size], pos % page_size, kv head, :]
 * for K and for V - the address rule lf_decode_paged_bf16 and lf_paged_gather_bf16 read with.
 * Pure data movement (bit-exact). A position the table has no entry for, or a page id outside
 * [0, n_pages), is reported as LF_DEV_BAD_PAGE in `status` and that row is not written (the
 * kernel never stores outside the pools). Rows of different sequences must not share a page. */
int lf_kv_append_bf16(const LfKvAppendArgs* args, void* stream);

/* 1 when the library was built with -DLF_DEBUG_BOUNDS (python -m loopfuse_b200.build
 * --debug-bounds -> liblf_sm100_dbg.so): every index that a kernel forms for a plain global
 * load or store - token, page slot, staged page-table entry, workspace row, output row - is then
 * compared with its range first; a violation writes LF_DEV_BOUNDS | (site << 8) to the call's
 * `status` word and the access is clamped or skipped, nothing traps. Stands in for
 * compute-sanitizer's memcheck where that tool cannot be used. 0 in the normal build. */
int lf_debug_bounds(void);

/* Elementwise out = a + b on bf16 [B, H, S, D] tensors (innermost stride 1, 16-byte aligned rows,
 * D % 8 == 0), each with its own element strides of (b, h, s); `out` may alias `a` or `b`. One
 * rounding to bf16, as the eager `Q + q_bias` and `scores @ V + out_bias` of the reference's
 * modified-attention test (tests/test_accuracy.py:177-181) have; the compiled front end uses it
 * for the query bias (before lf_prefill_bf16) and the output bias (after it). */
int lf_add_bf16(const void* a, const void* b, void* out, int32_t B, int32_t H, int32_t S,
                int32_t D, const int64_t* a_stride, const int64_t* b_stride,
                const int64_t* out_stride, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LF_SM100_H_ */
