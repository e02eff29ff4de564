/*
 * libbas — batch-shared block-sparse activation GEMM for LLM decoding on NVIDIA B200 (sm_100a).
 *
 *   Y[b, n] = sum over active 64-channel blocks j of  X[b, 64j:64j+64] . W[n, 64j:64j+64]
 *
 * One mask over 64-channel blocks of the input activation is shared by every row of the decode
 * batch; only the weight slabs of active blocks are read.  fp16 in, fp32 accumulate, fp16 out.
 *
 * This is the C ABI that a binding of the reference's Python operator module
 * (kernels/shared_mask_batched_triton_min_runtime.py) calls instead of launching Triton kernels.
 * All pointers named *_dev are device pointers on the current CUDA device, `stream` is a
 * cudaStream_t passed as void*, and every function returns a bas_status (0 = success).  No entry
 * point in the "device pointer" group allocates, synchronises or reads device memory on the host,
 * so all of them may be captured in a CUDA graph after one warm-up call.
 */
#ifndef BAS_H_
#define BAS_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define BAS_API __attribute__((visibility("default")))
#else
#define BAS_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define BAS_BLOCK_K 64   /* channels per activation block: INDEX_BLOCK_META_SIZE, kernels/...min_runtime.py:17 */
#define BAS_TILE_N 128   /* widest column sub-tile one kernel pass handles */
#define BAS_MAX_BLOCKS 4096 /* largest K/64 the kernels accept */
#define BAS_MAX_BATCH 64 /* largest decode batch of one call */

typedef enum bas_status {
  BAS_OK = 0,
  BAS_ERR_INVALID_ARGUMENT = 1, /* null pointer, non-positive size, misaligned pointer or stride */
  BAS_ERR_UNSUPPORTED = 2,      /* batch > BAS_MAX_BATCH, K/64 > BAS_MAX_BLOCKS, wrong GPU architecture */
  BAS_ERR_WORKSPACE = 3,        /* workspace missing or smaller than bas_gemm_workspace_bytes() */
  BAS_ERR_CUDA = 4,             /* a CUDA runtime or driver call failed; see bas_last_cuda_error() */
  BAS_ERR_DEVICE_FLAG = 5,      /* a kernel reported a bad block id or an expired wait (bas_read_device_status) */
  BAS_ERR_TOO_LARGE = 6         /* size beyond the fixed capacity of a no-allocation entry point */
} bas_status;

/* Bits of the device status word (first 4 bytes of every GEMM workspace). */
#define BAS_DEV_BAD_BLOCK_ID 1u  /* an id outside [0, K/64) was skipped */
#define BAS_DEV_WAIT_EXPIRED 2u  /* a bounded barrier wait ran out; the output is not valid */
/* With it the list kernel leaves a detail in the upper bits, for diagnosis (test for BAS_DEV_WAIT_EXPIRED itself):
 * bits 16-27 the index of the earliest call in which a wait ran out, bits 8-12 which wait of that call:
 * 0x100 a copy warp (a dependency or a ring slot), 0x200 an MMA-issuing warp, 0x400 an epilogue warp,
 * 0x800 / 0x1000 the exchange between ranks, on the rank that adds a tile / on a rank that receives it. */

typedef enum bas_score_kind {
  BAS_SCORE_NORM = 0,  /* mean_b ||x_b,block||_2 : scripts/bench_roundrobin_e2e_decode.py:103-105 */
  BAS_SCORE_ENERGY = 1, /* mean_b ||x_b,block||^2 : scripts/bench_alpaca_energy_budget_e2e.py:43-46 */
  BAS_SCORE_BF16 = 256, /* OR into score_kind: x holds bfloat16 instead of fp16 */
  /* OR into score_kind of bas_select_topk / bas_select_topk_weighted: the caller promises that no
   * kernel that can still be running when this call starts (the kernel preceding it in the stream,
   * and earlier ones where that kernel itself was allowed to start early) writes x_dev or touches
   * this call's outputs or workspace - e.g. the preceding kernel is the contraction of the PREVIOUS
   * step, launched without promises, reading the other of two alternating id buffers.  The
   * selection then scores while that kernel is still running and waits for it only before it
   * writes ids, count and byte map. */
  BAS_SCORE_INPUTS_STABLE = 512
} bas_score_kind;

BAS_API const char* bas_status_string(int status);
/* cudaError_t of the last failing CUDA call made by this library on the calling thread. */
BAS_API int bas_last_cuda_error(void);
/* Bound of the kernels' waits (barriers inside a CTA, counters between CTAs, words from other ranks)
 * for launches made from now on, process-wide: default about one second, accepted up to 10 s.  A
 * wait that runs out sets BAS_DEV_WAIT_EXPIRED and the kernel returns.  Tests shorten it to see that
 * path; a serving host may want it below its own watchdog. */
BAS_API int bas_set_wait_ms(double wait_ms);
/* Number of kernels this library has launched from this process (all threads). */
BAS_API unsigned long long bas_launch_count(void);

/* ---- weight prepack -------------------------------------------------------------------------
 * Replaces _get_prepacked_weight_block_major (kernels/...min_runtime.py:3133-3163): a one-time
 * repack of an nn.Linear weight W[N, K] (row stride ldw elements).  The reference packs to
 * [K/64, 64, N]; this library packs to its own layout [ceil(K/64)][N rounded up to 8][64]: per block,
 * one 128-byte row per output column with the 128-byte shared-memory swizzle pre-applied, so that
 * any range of output columns of a block is one contiguous chunk that lands in shared memory
 * ready for the tensor cores.  The packed tensor is opaque to callers, as it is in the reference. */
BAS_API size_t bas_packed_weight_bytes(int n, int k);
BAS_API int bas_pack_weight(const void* w_dev, int n, int k, int64_t ldw, void* packed_dev, void* stream);

/* ---- the contraction ------------------------------------------------------------------------
 * Replaces the launch sites of the reference's index-list and bitmap kernels and their split-K
 * pairs (kernels/...min_runtime.py:1124, :1288, :1310+:1334, :1400, :1417+:1441, :3331).
 *
 * The active set is given EITHER as an id list (ids_dev, k_host entries; if count_dev is non-null
 * the kernel reads the number of entries from device memory instead, k_host being an upper bound)
 * OR as a byte map (bitmap_dev[K/64], non-zero = active), the form the bitmap kernels consume
 * (kernels/...min_runtime.py:847); k_host is then only a hint of how many blocks are active
 * (0 = unknown), used to size the grid.  ids may be unsorted; they must be distinct.  An id outside
 * [0, ceil(K/64)) is skipped and flagged in the device status word.  An empty set writes zeros
 * (kernels/...min_runtime.py:1252-1254).
 *
 *   x_dev   fp16 [batch, K], row stride ldx elements (16-byte aligned rows)
 *   y_dev   fp16 [batch, N], row stride ldy elements, fully overwritten
 *   ws_dev  workspace of at least bas_gemm_workspace_bytes(batch, n) bytes, zero-filled once with
 *           bas_workspace_init().  It holds the device status word; the kernels keep all partial
 *           sums on chip, so calls may share it freely.
 * Every batch size runs the tcgen05 kernel unless bas_gemm_ex is asked for the CUDA-core one. */
BAS_API size_t bas_gemm_workspace_bytes(int batch, int n);
BAS_API int bas_workspace_init(void* ws_dev, size_t ws_bytes, void* stream);
BAS_API int bas_gemm(const void* x_dev, int64_t ldx, const void* packed_dev, const int32_t* ids_dev,
             const int32_t* count_dev, int k_host, const uint8_t* bitmap_dev, int batch, int k, int n,
             void* y_dev, int64_t ldy, void* ws_dev, size_t ws_bytes, void* stream);
/* As bas_gemm, with flags:
 *   bits 0-1  kernel family: 0 = chosen by batch size, 1 = CUDA-core kernel, 2 = tcgen05 kernel
 *   BAS_GEMM_IDS_STABLE  the caller promises that ids_dev is NOT written by the kernel that
 *             immediately precedes this call in the stream (a fixed mask, or one selected several
 *             launches earlier).  The kernel is launched with programmatic stream serialization;
 *             with this flag it starts streaming weight tiles while the previous kernel is still
 *             draining, and waits for it only before reading X and writing Y.  Without the flag
 *             only the kernel's own preamble overlaps.  Ignored when count_dev is given.
 *   BAS_GEMM_X_STABLE  (with BAS_GEMM_IDS_STABLE, tcgen05 kernel; ignored otherwise) the caller
 *             promises the same of x_dev: X was complete before the preceding kernel started
 *             (a resident input, or the X the preceding call of this library already read, as for
 *             q/k/v or gate/up of one layer).  Nothing the kernel reads then depends on the kernel
 *             before it: it streams and multiplies straight through and waits for that kernel only
 *             before its first store to Y.  A preceding call that carries the flag itself may have
 *             started before ITS predecessor finished: X must then not be that call's output
 *             either, and so on back to the last call launched without the flag.
 *             Such calls are given a small grid (one CTA per 128 output columns) so that several of
 *             them are resident at once: meant for calls launched back to back (one CUDA graph, or
 *             a launch loop that keeps ahead of the GPU); a call that runs alone takes about twice
 *             as long with the flag as without it.
 *   BAS_GEMM_NEXT_INDEPENDENT  (with the two flags above) a hint, not a promise: the call after
 *             this one will carry BAS_GEMM_X_STABLE too (a chain of independent calls).  Outputs of
 *             more than 9 472 columns at batches of up to 32 rows then run two 128-column passes per
 *             CTA on half as many CTAs, which pays only if the next calls do run beside this one.
 *   bits 8-10 cluster size of the tcgen05 kernel: 0 = chosen by batch size, else 1, 2 or 4 CTAs
 *             share the active blocks of one column range (reduced on chip, in rank order).
 *   BAS_GEMM_BF16  X, the packed weight and Y hold bfloat16 instead of fp16 (the reference's kernels
 *             take either, kernels/...min_runtime.py:21); tcgen05 kernel only.
 *   bits 12-14 copy/MMA warp pairs of the tcgen05 kernel: 0 = chosen by the ring size, else 2, 3
 *             or 4 (a tuning knob; results differ only in fp32 summation order).
 *   bits 16-23 upper bound on the CTAs of the tcgen05 kernel: 0 = chosen by the amount of work
 *             (a tuning knob).
 *   bit 24    bas_select_gemm only: select inside the contraction kernel whenever the shape has
 *             clusters, also where the two-launch chain is measured faster (a tuning knob). */
#define BAS_GEMM_IDS_STABLE 16
#define BAS_GEMM_BF16 32
#define BAS_GEMM_X_STABLE 64
#define BAS_GEMM_NEXT_INDEPENDENT 128
BAS_API int bas_gemm_ex(const void* x_dev, int64_t ldx, const void* packed_dev, const int32_t* ids_dev,
                const int32_t* count_dev, int k_host, const uint8_t* bitmap_dev, int batch, int k, int n,
                void* y_dev, int64_t ldy, void* ws_dev, size_t ws_bytes, int flags, void* stream);
/* Synchronous: copies the status word of a workspace to *flags_out (0 = clean) and clears it. */
BAS_API int bas_read_device_status(void* ws_dev, unsigned int* flags_out, void* stream);

/* ---- bitmap ---------------------------------------------------------------------------------
 * Replaces _build_active_k_bitmap (kernels/...min_runtime.py:1056-1061): u8[nb], 1 at active ids.
 * count_dev may be null (then k_host ids are used). */
BAS_API int bas_build_bitmap(const int32_t* ids_dev, const int32_t* count_dev, int k_host, int nb,
                     uint8_t* bitmap_dev, void* stream);

/* ---- per-step batch-shared mask selection ---------------------------------------------------
 * Replaces _select_active_blocks (scripts/bench_roundrobin_e2e_decode.py:90-113) and
 * _block_energy + _topk_active / _energy_budget_active
 * (scripts/bench_alpaca_energy_budget_e2e.py:43-62): one launch, no host synchronisation.
 * Scores are accumulated in fp64 from the exact fp16 (or, with BAS_SCORE_BF16, bfloat16) inputs; equal scores go to
 * the lower id, and a score that is not a number ranks above +infinity (the order of torch.topk and of a
 * descending torch.sort), so the ranking is a total order whatever X holds: exactly n_keep ids are written.
 * A budget whose total is not a number keeps every block.
 *
 *   ids_out_dev     int32 [>= n_keep] (top-k) or [>= K/64] (budget): ascending active ids
 *   count_out_dev   int32 [1]: number of ids written
 *   bitmap_out_dev  optional u8 [K/64]
 *   scores_out_dev  optional fp64 [K/64]: the batch-mean scores
 *   ws_dev          at least bas_select_workspace_bytes(K) bytes, zero-filled once with
 *                   bas_workspace_init()
 * bas_select_topk keeps n_keep blocks (callers compute n_keep = max(1, min(nb, round(density*nb)))).
 * bas_select_budget keeps the shortest descending-energy prefix reaching energy_keep of the total,
 * clamped to [min_keep, nb]. */
BAS_API size_t bas_select_workspace_bytes(int k);
BAS_API int bas_select_topk(const void* x_dev, int64_t ldx, int batch, int k, int n_keep, int score_kind,
                    int32_t* ids_out_dev, int32_t* count_out_dev, uint8_t* bitmap_out_dev,
                    double* scores_out_dev, void* ws_dev, size_t ws_bytes, void* stream);
BAS_API int bas_select_budget(const void* x_dev, int64_t ldx, int batch, int k, double energy_keep, int min_keep,
                      int32_t* ids_out_dev, int32_t* count_out_dev, uint8_t* bitmap_out_dev,
                      double* scores_out_dev, void* ws_dev, size_t ws_bytes, void* stream);
/* bas_select_topk with the two optional score modifiers of _select_active_blocks
 * (scripts/bench_roundrobin_e2e_decode.py:104-112, arguments block_score_scale and block_prior):
 *   chan_scale_dev  optional fp32 [>= 64 * (K/64)], 16-byte aligned: with it a block's score is
 *                   mean_b sum_i x[b,i]^2 * chan_scale[i], whatever score_kind says (as in the reference)
 *   block_mult_dev  optional fp32 [K/64]: factor on the batch-mean score.  The reference's
 *                   clamp(prior + eps, 1e-6) ** alpha is evaluated by the caller, once per prior.
 * With both null it is bas_select_topk. */
BAS_API int bas_select_topk_weighted(const void* x_dev, int64_t ldx, int batch, int k, int n_keep, int score_kind,
                             const float* chan_scale_dev, const float* block_mult_dev, int32_t* ids_out_dev,
                             int32_t* count_out_dev, uint8_t* bitmap_out_dev, double* scores_out_dev,
                             void* ws_dev, size_t ws_bytes, void* stream);
/* The same with score_flags = 0 or BAS_SCORE_BF16. */
BAS_API int bas_select_budget_ex(const void* x_dev, int64_t ldx, int batch, int k, double energy_keep, int min_keep,
                         int score_flags, int32_t* ids_out_dev, int32_t* count_out_dev, uint8_t* bitmap_out_dev,
                         double* scores_out_dev, void* ws_dev, size_t ws_bytes, void* stream);

/* bas_select_budget_ex with the dense fallback of _patch_adaptive
 * (scripts/bench_alpaca_energy_budget_e2e.py:104-109) taken on the device: when the budget keeps more
 * than full_above blocks, every block is kept (count = K/64), so that the contraction that follows
 * computes the dense product without the host having to read the count. */
BAS_API int bas_select_budget_capped(const void* x_dev, int64_t ldx, int batch, int k, double energy_keep, int min_keep,
                             int full_above, int score_flags, int32_t* ids_out_dev, int32_t* count_out_dev,
                             uint8_t* bitmap_out_dev, double* scores_out_dev, void* ws_dev, size_t ws_bytes,
                             void* stream);

/* ---- selection and contraction in one call -------------------------------------------------
 * The chain of _sparse_linear (scripts/bench_roundrobin_e2e_decode.py:179-284): select the batch's
 * blocks, then multiply.  Where the contraction runs in clusters and the scoring is small (up to
 * about 256 (block, row) pairs per CTA: batches of a few rows) the selection runs inside the
 * contraction kernel - every cluster scores X for itself, its CTAs sharing the blocks - so the chain
 * is one launch; elsewhere it is the two launches bas_select_topk / bas_select_budget_ex + bas_gemm,
 * which is the faster form there.  Same ids, same sums either way.
 *   energy_keep < 0   top-k of n_keep blocks by score_kind (| BAS_SCORE_BF16 with BAS_GEMM_BF16)
 *   energy_keep >= 0  energy budget, at least n_keep blocks
 *   ids_out_dev [>= K/64], count_out_dev [1]  required; bitmap_out_dev, scores_out_dev optional
 *   flags: BAS_GEMM_BF16 and the tuning bits of bas_gemm_ex */
BAS_API int bas_select_gemm(const void* x_dev, int64_t ldx, const void* packed_dev, int batch, int k, int n, int n_keep,
                            int score_kind, double energy_keep, void* y_dev, int64_t ldy, int32_t* ids_out_dev,
                            int32_t* count_out_dev, uint8_t* bitmap_out_dev, double* scores_out_dev,
                            void* gemm_ws_dev, size_t gemm_ws_bytes, void* select_ws_dev, size_t select_ws_bytes,
                            int flags, void* stream);

/* ---- a list of contractions as one launch ---------------------------------------------------
 * The call pattern of a decode step: the reference patches every nn.Linear of the model and runs
 * them one after the other, 224 per token for Llama-2-7B (scripts/bench_roundrobin_e2e_decode.py:331-503),
 * and its benchmark adds the 224 per-projection times up per step
 * (scripts/bench_perstep_actual_kernel_speedup.py:268-293).  A bas_list holds such a sequence of
 * bas_gemm calls and runs it as ONE persistent kernel: the CTAs walk the list, the weight tiles of
 * a call are fetched while the call before it is still being finished (weights never depend on
 * it), and only a call's activations wait - for the call named in depends_on, on a counter in
 * device memory.  Same sums as the single calls, same rounding; results do not depend on timing.
 *
 *   depends_on  index of an EARLIER call of the list that must be complete before x_dev is read
 *               (normally the call that writes x_dev), or -1: x_dev is complete before the launch.
 *               A call may overwrite a buffer that an earlier call reads only if it depends,
 *               directly or through other calls, on that earlier call.
 *   id lists, counts and byte maps must be complete before the launch (they may change between
 *   runs); K / 64 of a call is at most BAS_LIST_MAX_BLOCKS, a list holds at most BAS_LIST_MAX_CALLS.
 *   flags of bas_list_create: BAS_GEMM_BF16 and the tuning bits 8-10 (cluster size), 12-14 (warp
 *   pairs) and 16-23 (upper bound on the CTAs) of bas_gemm_ex.
 *
 * Selection inside the list (a decode step computes every mask from the activation it is about to
 * multiply: scripts/bench_roundrobin_e2e_decode.py:90-113, 331-360).  An entry with op = BAS_LIST_SELECT is
 * bas_select_topk as part of the launch: x_dev / ldx / batch / k (a multiple of 64) describe X, k_host is the
 * number of blocks to keep, score_kind the score, depends_on the call that writes X; every other field is
 * zero.  Its CTAs score the blocks with the arithmetic of bas_select_topk (same bits) as soon as X is
 * complete and rank them - (score descending, id ascending), NaN first.  A contraction whose mask_entry names
 * that entry (same X: same batch, same depends_on) picks the verdicts up at its call boundary and runs with the
 * kept blocks in ascending order, exactly as if bas_select_topk's list had been passed; its weights cannot be
 * fetched before the mask exists, so such a call costs more than a call whose mask was known before the launch.
 * Several calls may use one entry (q, k and v; gate and up).  Top-k only; one CTA per column range only.
 *
 * A SELECT entry over a K-sharded activation (bas_list_create_tp; shape_flags = BAS_LIST_SELECT_SHARDED): x_dev
 * holds this rank's blocks only, mask_block0 is their first block in the whole input and n_host the blocks of the
 * whole input (at most 1024), k_host still counts blocks of the whole input.  Every rank scores its own blocks, the
 * scores travel to all ranks through the group's exchange area and a block is kept by its rank among ALL blocks,
 * so that every rank runs with its part of one global top-k, as the unsharded model would (the 64 to 172 scores
 * that have to be gathered before a global selection).  The contractions that run with such an entry are the
 * row-parallel calls over that same shard (mask_block0 as the entry's).  The entries share one region of the
 * exchange area: an entry must depend, directly or through other calls, on the last row-parallel call before it,
 * and a row-parallel call must lie between two such entries.
 *
 * Output-block sparsity and compact operands (the reference's 2-D kernels and their compact chaining of
 * gate/up into down, kernels/shared_mask_batched_triton_min_runtime.py:2289-2386, 2473-2558, 3411-3467,
 * 3498-3850).  With n_ids_dev a call computes only the output blocks named there (64 columns each, n_host ids in
 * [0, ceil(n / 64)), complete before the launch, any order): Y[:, 64 o .. 64 o + 63] for every listed o, the other
 * columns of y are not touched - or, with BAS_LIST_OUT_COMPACT, block q of the list goes to columns 64 q .. of a
 * y that is n_host * 64 wide.  BAS_LIST_X_COMPACT: x_dev holds only the active input blocks, in the order of the
 * id list (block i of X belongs to ids_dev[i]; k stays the K of the weight), which is what a compact output of
 * the call before is.  Not with row_parallel, not with clusters.  An id out of range sets BAS_DEV_BAD_BLOCK_ID.
 *
 * bas_list_create allocates a few hundred bytes per call of device memory and uploads the
 * descriptors (synchronous); bas_list_run only launches, so it may be captured in a CUDA graph.
 * Runs of one list must not overlap on the GPU.  bas_list_read_status is bas_read_device_status for
 * the list's own status word.  A run that reported BAS_DEV_WAIT_EXPIRED leaves the list's counters
 * inconsistent: call bas_list_reset (synchronous) before the next run.
 * bas_list_set_wait changes the bound of the kernel's waits (default about one second) and, for
 * tests of the expiry path only, names a call whose dependency is never seen complete (-1: none). */
#define BAS_LIST_MAX_BLOCKS 1024
#define BAS_LIST_MAX_CALLS 4096
#define BAS_LIST_GEMM 0
#define BAS_LIST_SELECT 1
#define BAS_LIST_OUT_COMPACT 1
#define BAS_LIST_X_COMPACT 2
#define BAS_LIST_SELECT_SHARDED 4
typedef struct bas_list_call {
  const void* x_dev;
  int64_t ldx;
  const void* packed_dev;
  const int32_t* ids_dev;
  const int32_t* count_dev;
  const uint8_t* bitmap_dev;
  void* y_dev;
  int64_t ldy;
  int32_t k_host, batch, k, n;
  int32_t depends_on;
  int32_t row_parallel;   /* bas_list_create_tp only: 1 = x / packed are this rank's K-shard, y receives the sum over the ranks */
  int32_t op;             /* BAS_LIST_GEMM (0) or BAS_LIST_SELECT */
  int32_t mask_entry;     /* GEMM: 1 + index of the earlier BAS_LIST_SELECT entry whose mask it runs with; 0: ids / count / byte map above */
  int32_t mask_block0;    /* GEMM with mask_entry: the block of that mask which is block 0 of this call (a K-shard); else 0.
                             SELECT with BAS_LIST_SELECT_SHARDED: the first block of this rank's shard in the whole input */
  int32_t score_kind;     /* SELECT: BAS_SCORE_NORM or BAS_SCORE_ENERGY */
  int32_t* ids_out_dev;   /* GEMM with mask_entry, optional: receives the kept ids of the whole mask, ascending (k_host of the entry) */
  const int32_t* n_ids_dev; /* GEMM, optional: only these 64-column output blocks are computed (see below); n_host of them */
  int32_t n_host;         /* (SELECT with BAS_LIST_SELECT_SHARDED: the blocks of the whole input) */
  int32_t shape_flags;    /* GEMM: BAS_LIST_OUT_COMPACT | BAS_LIST_X_COMPACT; SELECT: BAS_LIST_SELECT_SHARDED */
} bas_list_call;
typedef struct bas_list bas_list;
BAS_API int bas_list_create(bas_list** out, const bas_list_call* calls, int n_calls, int flags);
/* A list for one rank of a tensor-parallel group (bas_tp_*, connected): calls marked row_parallel add
 * their outputs over the ranks inside the kernel - every rank sends a column tile's fp32 partials to the
 * one rank that owns the tile, which adds them in rank order, rounds once and sends the 16-bit results to
 * the others; identical bits on all ranks - so a sharded decode step is one launch per rank.  Every rank
 * must create the same list (same shapes and order; its own shards) and run it equally often; a
 * row-parallel call must depend, directly or through other calls, on the row-parallel call before it;
 * one CTA per column range only.  A wait that runs out: as for bas_gemm_allreduce, the group is dead. */
typedef struct bas_tp bas_tp;
BAS_API int bas_list_create_tp(bas_list** out, const bas_list_call* calls, int n_calls, int flags, bas_tp* tp);
BAS_API int bas_list_run(bas_list* l, void* stream);
BAS_API int bas_list_read_status(bas_list* l, unsigned int* flags_out, void* stream);
BAS_API int bas_list_reset(bas_list* l);
BAS_API int bas_list_set_wait(bas_list* l, double wait_ms, int never_ready_call);
/* ctas, cluster size, ring slots and warp pairs of the list's kernel (any pointer may be null). */
BAS_API int bas_list_info(const bas_list* l, int* ctas, int* cluster, int* slots, int* pairs);
BAS_API void bas_list_destroy(bas_list* l);

/* ---- selection for callers that must not allocate -------------------------------------------
 * No counterpart in the reference.  Same result as bas_select_topk, but the caller passes no
 * workspace and the library allocates nothing: the kernel's scratch (one fp64 score per block and
 * an arrival counter, BAS_NOALLOC_MAX_BLOCKS * 8 + 256 bytes) is a fixed device array inside the
 * library image, which every GPU that loads libbas keeps until the process exits.
 * It is meant for hosts that have handed every spare byte of device memory to a pool of their own
 * (an inference server that sizes its KV-cache arena to fill the GPU) or whose decode loop runs
 * under a rule that no CUDA allocation call may happen after start-up: for them cudaMalloc either
 * fails or stalls the device, so a workspace cannot be conjured at call time.
 *  - K / 64 above BAS_NOALLOC_MAX_BLOCKS returns BAS_ERR_TOO_LARGE.
 *  - The first call on each device looks up the array's device address (the device must be
 *    current); make that first call before starting any stream capture.
 *  - All calls on a device share the one array: two calls that overlap on the GPU (different
 *    streams) race on it.  Calls on one stream are safe back to back. */
#define BAS_NOALLOC_MAX_BLOCKS 1024   /* K up to 65 536 */
BAS_API int bas_select_topk_noalloc(const void* x_dev, int64_t ldx, int batch, int k, int n_keep, int score_kind,
                                    int32_t* ids_out_dev, int32_t* count_out_dev, uint8_t* bitmap_out_dev,
                                    double* scores_out_dev, void* stream);

/* ---- row-parallel contraction with the sum over ranks formed in the kernel -------------------
 * No counterpart in the reference (it is single-GPU).  For the o / down projections of a
 * tensor-parallel layer: every rank (one process per GPU of one box) multiplies its K-shard and
 * the partial outputs are added inside the contraction kernel, through an exchange area that each
 * rank maps into its peers (CUDA IPC, plain peer stores over NVLink).  CTA c of every rank sends
 * its fp32 partial to every rank's area as 64-bit words {value, call number}, polls (bounded, about
 * a second) its own area until the words of all ranks carry the current call number, and adds them
 * in rank order: the result is identical on all ranks and does not depend on timing; one NVLink
 * traversal, no flags or fences.  A wait that runs out sets BAS_DEV_WAIT_EXPIRED and leaves Y of
 * that CTA unwritten; the ranks' call numbers are out of step from then on, so the group is dead:
 * disconnect and destroy it on every rank and create a new one.  All ranks must issue the same sequence of bas_gemm_allreduce calls on a
 * group (same batch and n per call, n at most the group's); calls on one group must not overlap
 * on a GPU.
 *
 *   bas_tp_create   allocates and zeroes this rank's area for outputs of up to max_batch x n
 *   bas_tp_handle   writes the area's BAS_TP_HANDLE_BYTES-byte inter-process handle
 *   bas_tp_connect  takes all ranks' handles (world x BAS_TP_HANDLE_BYTES, rank order; the caller
 *                   gathers them with whatever transport it has) and maps the peers' areas; every
 *                   rank must have returned from it before the first bas_gemm_allreduce
 *   bas_gemm_allreduce  bas_gemm_ex with k = this rank's K-shard; y receives the full sum
 *   bas_tp_disconnect unmaps the peers' areas; bas_tp_destroy does that too and frees this rank's
 *                   own area, which no peer may still have mapped: disconnect on every rank, meet
 *                   (a barrier of the caller's), then destroy */
#define BAS_TP_HANDLE_BYTES 64
#define BAS_TP_MAX_RANKS 8
BAS_API int bas_tp_create(bas_tp** out, int rank, int world, int max_batch, int n);
BAS_API int bas_tp_handle(bas_tp* tp, void* handle_out);
BAS_API int bas_tp_connect(bas_tp* tp, const void* handles);
BAS_API int bas_tp_disconnect(bas_tp* tp);
BAS_API void bas_tp_destroy(bas_tp* tp);
BAS_API int bas_gemm_allreduce(bas_tp* tp, const void* x_dev, int64_t ldx, const void* packed_dev,
                               const int32_t* ids_dev, const int32_t* count_dev, int k_host,
                               const uint8_t* bitmap_dev, int batch, int k, int n, void* y_dev, int64_t ldy,
                               void* ws_dev, size_t ws_bytes, int flags, void* stream);

/* ---- host-buffer operator -------------------------------------------------------------------
 * The call pattern of _sparse_linear (scripts/bench_roundrobin_e2e_decode.py:179-284) for a caller
 * whose activations live in host memory: a handle owns the packed weight, the device staging
 * buffers, a workspace and a stream.  forward copies X host->device, selects the mask on the
 * device (or takes the caller's ids), runs the contraction, copies Y (and the ids) back and waits.
 * w_host is fp16 [n, k] row-major.  x_host/y_host are fp16 [batch, k] / [batch, n]. */
typedef struct bas_linear bas_linear;
BAS_API int bas_linear_create(bas_linear** out, const void* w_host, int n, int k, int max_batch);
BAS_API int bas_linear_forward_host(bas_linear* h, const void* x_host, int batch, int n_keep, int score_kind,
                            void* y_host, int32_t* ids_host_out);
BAS_API int bas_linear_forward_host_ids(bas_linear* h, const void* x_host, int batch, const int32_t* ids_host,
                                int n_ids, void* y_host);
/* bas_linear_forward_host in two halves: submit enqueues the copies and kernels on the handle's own
 * stream and returns; wait blocks until they are done and fills y_host / ids_host_out.  One forward
 * may be in flight per handle; forwards submitted on different handles overlap (copies of one with
 * kernels of another).  x_host must stay untouched, and y_host / ids_host_out unread, until wait
 * returns.  Buffers that are page-locked (cudaMallocHost, cudaHostRegister) are copied from and to
 * directly; others go through the handle's pinned staging buffers. */
BAS_API int bas_linear_submit_host(bas_linear* h, const void* x_host, int batch, int n_keep, int score_kind,
                                   void* y_host, int32_t* ids_host_out);
BAS_API int bas_linear_wait(bas_linear* h);
BAS_API void bas_linear_destroy(bas_linear* h);

/* ---- host-buffer operator for a whole step -------------------------------------------------
 * The call pattern of the patched model's token loop (scripts/bench_roundrobin_e2e_decode.py:515-548:
 * every linear of a step runs _sparse_linear, :179-284) for a caller whose activations live in host
 * memory, taken a STEP at a time: bas_step_submit enqueues, on a stream of the step's slot, the
 * upload of every call's X, the device-side top-k selections, ONE list launch for all contractions
 * and the download of every Y and id list, and returns; bas_step_wait blocks until the oldest
 * submitted step is done.  Up to `depth` steps are in flight, so the copies of one step run beside
 * the kernels of another; a step that recurs with the same page-locked buffers is replayed as one
 * CUDA-graph launch.  Calls that name the same w_host (fp16 [n, k] row-major) share one packed copy.
 * x_host[c] is fp16 [batch_c, k_c], y_host[c] fp16 [batch_c, n_c], ids_host_out (optional, entries may
 * be null) receives n_keep_c ascending ids per call; all must stay valid until the step's wait returns. */
typedef struct bas_step_call {
  const void* w_host;
  int32_t n, k, batch, n_keep, score_kind, reserved;
} bas_step_call;
typedef struct bas_step bas_step;
BAS_API int bas_step_create(bas_step** out, const bas_step_call* calls, int n_calls, int depth);
BAS_API int bas_step_submit(bas_step* s, const void* const* x_host, void* const* y_host, int32_t* const* ids_host_out);
BAS_API int bas_step_wait(bas_step* s);
BAS_API void bas_step_destroy(bas_step* s);

#ifdef __cplusplus
}
#endif
#endif /* BAS_H_ */
