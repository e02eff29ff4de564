// Swapped-operand tcgen05 kernel for decode batches of 1..64 rows.
//
// Work split: the output columns are cut into one contiguous range per CTA (or per cluster); a CTA
// walks the active blocks and keeps the whole [columns x batch] result of its range in tensor
// memory, so no CTA ever needs another grid-mate's partial sums through global memory.  With a
// cluster of 2 or 4 CTAs the active blocks of one (wider) range are dealt out round-robin to the
// cluster's CTAs and their fp32 partials are added through distributed shared memory in rank
// order; this divides the activation traffic per SM by the cluster size and fills the MMA's 128
// rows, which is what large batches need.
//
// Per active block j and column sub-tile (up to 128 columns starting at n0):
//     D[128 x Bpad] (TMEM, fp32) += Wchunk[cols x 64] (smem, K-major, 128B swizzle) * Xtile[Bpad x 64]^T
// Wchunk is rows n0.. of block j in the packed layout: contiguous, stored pre-swizzled, fetched by
// one 1-D bulk copy.  Xtile comes straight from X[batch, K] by a 2-D tensor-map copy with the same
// swizzle; rows past the batch and channels past K arrive as zeros.  The MMA always spans 128 rows:
// rows past the chunk read whatever the ring holds there and only feed accumulator lanes that are
// never stored.
//
// Roles: warps 0..3 issue copies (warp 0 first stages the id list), warps 4..7 issue MMAs (one
// elected thread each, one accumulator each), warps 8..15 drain the accumulators (tcgen05.ld), add
// them and store or, in cluster mode, push them to the owning CTA.  All waits are bounded mbarrier
// waits; TMEM is released on every path.
//
// Calls that declared their id list and X stable (nothing they read depends on the kernel before
// them) run on a small grid - one CTA per 128-column range, wide outputs optionally two passes per CTA
// with accumulator columns per pass - and wait for their predecessor only before they store, so
// that several calls of a stream are resident at once.
//
// Two variants are instantiated beside the plain kernel: TP sends the result as fp32 partials to the
// other ranks of a box and adds theirs (row-parallel linears), SEL selects the batch's mask itself
// before multiplying (cluster modes, small batches).
//
// Replaces the reference's bitmap/index-list tl.dot kernels and their split-K
// pairs (kernels/shared_mask_batched_triton_min_runtime.py:814-874, 1150-1216, 1956-1988).
#include "bas_kernels.cuh"

#include <cudaTypedefs.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

namespace bas {

namespace {

// The ring is worked by P = GemmParams::issuers pairs (2..4) of one copy-issuing warp and one
// MMA-issuing warp: pair w owns ring groups w, w+P, ... and, the slot count being a multiple of P,
// always the same slots.  A pair is thus an in-order ring of its own, and no mbarrier is ever waited
// on by a thread that could be more than one phase away from it.
constexpr int kProducers = 4;           // copy-issuing warps available
constexpr int kIssuers = 4;             // MMA-issuing warps available; each owns one accumulator
constexpr int kEpiWarp0 = kProducers + kIssuers;   // first epilogue warp (a multiple of 4: TMEM lane quarters)
constexpr int kEpiThreads = 256;   // two sets of four warps
constexpr int kUmmaThreads = 32 * kEpiWarp0 + kEpiThreads;
constexpr int kTmemCols = 64 * kIssuers;   // one 64-column fp32 accumulator per issuer
constexpr int kMmaSpanBytes = 128 * kRowBytes;   // an M=128 operand read spans 16 KiB from the slot base

// XOR applied to the index of a four-slot group within a column of the cluster receive buffer
// (nbi slots = nbi * 4 bytes per column): makes 16-byte accesses of eight neighbouring columns fall
// into eight different bank groups.  Group counts that are not powers of two are left alone.
__device__ __forceinline__ int red_swizzle(int nbi, int r) {
  return nbi == 32 ? (r & 7) : nbi == 16 ? ((r >> 1) & 3) : nbi == 8 ? ((r >> 2) & 1) : 0;
}

// This rank's partial of one output element, sent to every rank of a tensor-parallel group (its own
// included) as one 64-bit word {value, call number}.  Kept out of line: the exchange is the rare
// path and must not bloat the epilogue's unrolled store loops.
__device__ __noinline__ void tp_send_word(const TpExchange& tp, unsigned int epoch, size_t slot, int row, int col, float v) {
  const unsigned long long word = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
  const size_t off = slot + (size_t)row * (size_t)tp.ldp + (size_t)col;
#pragma unroll 1
  for (int q = 0; q < tp.world; ++q) st_relaxed_sys_u64((unsigned long long*)tp.area[q] + off, word);
}

struct UmmaSmemHeader {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full;      // every issuer has finished the sub-tile (kIssuers arrivals)
  uint64_t acc_empty;     // the epilogue has drained the accumulators (4 arrivals)
  uint64_t ids_ready;
  uint32_t tmem_base;
  int k_act;
  int abort_flag;
  int sel_keep;               // in-kernel selection: blocks kept
  int sel_warp_cnt[kUmmaThreads / 32];
  long long t0;   // diagnostic builds: clock at kernel start
};

inline size_t umma_ids_bytes(int nb) { return ((size_t)nb * 2 + 127) / 128 * 128; }
inline size_t umma_fixed_smem(int nb) {
  return 1024 /*alignment slack*/ + (sizeof(UmmaSmemHeader) + 127) / 128 * 128 + umma_ids_bytes(nb) + 1024;
}

// Bytes of scratch the in-kernel selection needs in the (not yet used) ring area: scores, ranks and
// rank order of all blocks, then the per-(block, row) scores of this CTA's share of the blocks.
inline size_t fused_select_scratch(int nb_sel, int cluster, int batch) {
  const size_t per_block = 2 * sizeof(double) + 2 * sizeof(int);
  const size_t mine = (size_t)(nb_sel + cluster - 1) / cluster;
  return ((size_t)nb_sel * per_block + 15) / 16 * 16 + mine * (size_t)batch * sizeof(double);
}

// The batch-shared mask selection of select_kernel (same arithmetic: fp64 sums of exact squares, rows
// added in order, ties to the lower id), run by one cluster for itself.  CTA `crank` scores blocks
// crank, crank + C, ...; the scores go to every CTA of the cluster through distributed shared memory;
// then every CTA ranks all blocks and compacts the kept ids, ascending, into s_ids.  Returns the
// number kept.  All threads of the CTA (and all CTAs of the cluster) must call it.
__device__ __forceinline__ int fused_select(const GemmParams& p, uint8_t* scratch, uint16_t* s_ids, int* s_warp_cnt,
                                            int* s_keep, int crank, int C, int tid, int nthreads,
                                            [[maybe_unused]] long long t0) {
  const int nb = p.sel.nb_sel, batch = p.batch;
  const bool bf16 = (p.flags & kFlagBf16) != 0;
  double* s_score = (double*)scratch;
  unsigned long long* s_key = (unsigned long long*)(s_score + nb);   // ranking keys (score_key)
  int* s_rank = (int*)(s_key + nb);
  int* s_order = s_rank + nb;
  double* s_pair = (double*)(scratch + ((size_t)nb * (2 * sizeof(double) + 2 * sizeof(int)) + 15) / 16 * 16);
  const int lane = tid & 31, warp = tid >> 5;
  const int nmine = (nb > crank) ? (nb - crank + C - 1) / C : 0;

  // ---- scores of this CTA's blocks: 8 lanes per (block, row) pair, 16 bytes per lane; four pairs
  // per lane group and round, loaded together so that their latencies overlap ----
  const int sub = tid & 7, grp = tid >> 3;
  const int pairs = nmine * batch;
  const int groups = nthreads / 8;
  for (int base = 0; base < pairs; base += 4 * groups) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int pr = base + u * groups + grp;
      v[u] = make_uint4(0u, 0u, 0u, 0u);
      if (pr < pairs) {
        const int jj = pr / batch, b = pr - jj * batch;
        v[u] = __ldg((const uint4*)(p.x + (size_t)b * p.ldx + (size_t)(crank + jj * C) * kBlockK) + sub);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int pr = base + u * groups + grp;
      double e = 0.0;
      if (bf16) {
        const unsigned int* wds = (const unsigned int*)&v[u];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const double lo = (double)__uint_as_float(wds[q] << 16), hi = (double)__uint_as_float(wds[q] & 0xffff0000u);
          e += lo * lo;
          e += hi * hi;
        }
      } else {
        const __half2* h = (const __half2*)&v[u];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __half22float2(h[q]);
          e += (double)(f.x * f.x);
          e += (double)(f.y * f.y);
        }
      }
      e += __shfl_xor_sync(0xffffffffu, e, 1);
      e += __shfl_xor_sync(0xffffffffu, e, 2);
      e += __shfl_xor_sync(0xffffffffu, e, 4);
      if (pr < pairs && sub == 0) s_pair[pr] = (p.sel.score_kind == BAS_SCORE_NORM) ? sqrt(e) : e;
    }
  }
  __syncthreads();
  if (tid == 0) BAS_TRACE_SET(20, BAS_TRACE_CLOCK() - t0);   // pair scores done
  const uint32_t score_base = smem_u32(s_score);
  for (int jj = tid; jj < nmine; jj += nthreads) {
    double sum = 0.0;
    for (int b = 0; b < batch; ++b) sum += s_pair[jj * batch + b];   // batch rows in order
    const double score = sum / (double)batch;
    const int j = crank + jj * C;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (q < C) dsmem_st_f64(dsmem_addr(score_base + (uint32_t)j * 8u, (uint32_t)q), score);
  }
  cluster_sync_all();   // every CTA of the cluster now holds every score
  if (tid == 0) BAS_TRACE_SET(21, BAS_TRACE_CLOCK() - t0);   // scores exchanged

  // ---- rank all blocks: four threads per block, on the same totally ordered keys as select_kernel
  // (integer compares are also far cheaper than fp64 ones) ----
  for (int j = tid; j < nb; j += nthreads) s_key[j] = score_key(s_score[j]);
  __syncthreads();
  const unsigned long long* s_bits = s_key;
  for (int j0 = 0; j0 < nb; j0 += nthreads / 4) {
    const int j = j0 + (tid >> 2), quad = tid & 3;
    int rank = 0;
    if (j < nb) {
      const unsigned long long sj = s_bits[j];
      for (int i = quad; i < nb; i += 4) {
        const unsigned long long si = s_bits[i];
        rank += (si > sj || (si == sj && i < j)) ? 1 : 0;
      }
    }
    rank += __shfl_xor_sync(0xffffffffu, rank, 1);
    rank += __shfl_xor_sync(0xffffffffu, rank, 2);
    if (j < nb && quad == 0) {
      s_rank[j] = rank;
      s_order[rank] = j;
    }
  }
  __syncthreads();
  if (tid == 0) BAS_TRACE_SET(22, BAS_TRACE_CLOCK() - t0);   // ranked
  if (tid == 0) {
    int keep = p.sel.n_keep;
    if (p.sel.mode == 2) {
      // energy budget: shortest descending prefix whose sum reaches energy_keep of the total
      double total = 0.0;
      for (int r = 0; r < nb; ++r) total += s_score[s_order[r]];
      const double thresh = p.sel.energy_keep * total;
      double cum = 0.0;
      int kk = nb;
      for (int r = 0; r < nb; ++r) {
        cum += s_score[s_order[r]];
        if (cum >= thresh) {
          kk = r + 1;
          break;
        }
      }
      keep = max(p.sel.n_keep, min(nb, kk));
    }
    *s_keep = min(max(keep, 0), nb);
  }
  __syncthreads();
  const int keep = *s_keep;
  // ---- ascending compaction of the kept ids; CTA 0 also writes the caller's outputs ----
  const bool writer = blockIdx.x == 0;
  int running = 0;
  for (int base = 0; base < nb; base += nthreads) {
    const int j = base + tid;
    const bool kept = (j < nb) && (s_rank[j] < keep);
    if (writer && j < nb) {
      if (p.sel.bitmap_out != nullptr) p.sel.bitmap_out[j] = kept ? 1 : 0;
      if (p.sel.scores_out != nullptr) p.sel.scores_out[j] = s_score[j];
    }
    const unsigned m = __ballot_sync(0xffffffffu, kept);
    if (lane == 0) s_warp_cnt[warp] = __popc(m);
    __syncthreads();
    int off = running;
    for (int w = 0; w < warp; ++w) off += s_warp_cnt[w];
    const int pos = off + __popc(m & ((1u << lane) - 1u));
    if (kept && pos < keep) {
      s_ids[pos] = (uint16_t)j;
      if (writer && p.sel.ids_out != nullptr) p.sel.ids_out[pos] = j;
    }
    for (int w = 0; w < nthreads / 32; ++w) running += s_warp_cnt[w];
    __syncthreads();
  }
  if (writer && tid == 0 && p.sel.count_out != nullptr) *p.sel.count_out = keep;
  if (tid == 0) BAS_TRACE_SET(23, BAS_TRACE_CLOCK() - t0);   // list compacted
  return keep;
}

// TP: the row-parallel variant that exchanges partial sums with the other ranks of a box instead of
// storing Y directly (a template parameter, so that the plain kernel carries none of that code).
// SEL: the variant that selects the mask itself (cluster modes, not combined with TP).
template <int BPAD, bool TP, bool SEL>
__global__ void __launch_bounds__(kUmmaThreads, 1)
    umma_colsplit_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap xmap) {
  const bool bf16 = (p.flags & kFlagBf16) != 0;
  // operand formats: bits 7-9 (A) and 10-12 (B) of the instruction descriptor, 0 = fp16, 1 = bf16
  const uint32_t kIdesc = umma_idesc_f16(128, BPAD) | (bf16 ? ((1u << 7) | (1u << 10)) : 0u);
  constexpr int kXTileBytes = BPAD * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sp = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  UmmaSmemHeader* hdr = (UmmaSmemHeader*)sp;
  sp += (sizeof(UmmaSmemHeader) + 127) / 128 * 128;
  uint16_t* s_ids = (uint16_t*)sp;
  sp += ((size_t)p.nb * 2 + 127) / 128 * 128;
  float* s_red = (float*)sp;   // cluster mode: partials pushed here by the cluster's CTAs, [source rank][row slot][128]
  if (p.cluster > 1) sp += (size_t)BPAD * kTileN * sizeof(float);
  uint8_t* s_stage = (uint8_t*)(((uintptr_t)sp + 1023) & ~(uintptr_t)1023);  // swizzle atoms need 1 KiB alignment
  const int S = p.stages, G = p.group;
  const int tile_bytes = p.wslot + kXTileBytes;   // multiple of 1024
  const int stage_bytes = G * tile_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &hdr->abort_flag;
  BAS_TRACE_LAUNCH_BEGIN();

  // The id list may be the previous kernel's output unless the caller declared it stable; so may X
  // unless declared stable too; Y always waits for the previous kernel.  A stable list is requested
  // right away, so that its load latency runs under the set-up below.
  const bool early_ids = !SEL && (p.flags & kFlagStableIds) != 0 && p.count_dev == nullptr;
  // With X stable as well nothing this kernel reads depends on the kernel before it: copies and MMAs
  // run straight through, and only the epilogue waits, before the first store to Y.
  const bool early_x = !TP && early_ids && (p.flags & kFlagStableX) != 0;
  // Where the launcher says so the wait is the last thing before a store: the accumulators are read out
  // and added first, so that what follows the predecessor's completion - the serial link of a chain
  // of calls - is short.
  const bool late_wait = early_x && (p.flags & kFlagLateWait) != 0;
  int first_ids[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (warp == 0 && early_ids)
    warp_load_id_batch(p.ids, p.bitmap, p.bitmap != nullptr ? p.nb : p.k_host, 0, lane, first_ids);

  if (tid < S) {
    mbar_init(&hdr->full[tid], 1);
    mbar_init(&hdr->empty[tid], 1);
    fence_barrier_init();
  } else if (tid == 64) {
    mbar_init(&hdr->acc_full, p.issuers);
    mbar_init(&hdr->acc_empty, kEpiThreads / 32);
    mbar_init(&hdr->ids_ready, 1);
    hdr->abort_flag = 0;
    hdr->k_act = 0;
    hdr->t0 = BAS_TRACE_CLOCK();
    fence_barrier_init();
    prefetch_tensormap(&xmap);
  }
  if (warp == kEpiWarp0) {
    tmem_alloc(&hdr->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = hdr->tmem_base;
  if (tid == 0) {
    BAS_TRACE_SET(8, BAS_TRACE_CLOCK() - hdr->t0);     // preamble done
    BAS_TRACE_SET(13, p.cluster * 1000000 + p.issuers * 1000 + p.stages * 10 + p.group);
    BAS_TRACE_SET(14, p.ranges);
  }

  // this CTA's columns and its share of the active list
  const int C = p.cluster;
  const int rank = (C > 1) ? (int)cluster_ctarank() : 0;
  const int range = blockIdx.x / C;
  const int units = p.npad >> 3;
  const int n0 = col_begin(range, units, p.ranges), n1 = col_begin(range + 1, units, p.ranges);
  const int width = n1 - n0;
  constexpr int TW = kTileN;                        // columns per pass
  const int n_sub = (width + TW - 1) / TW;

  if (SEL) {
    // Mask selection by this cluster, for itself.  X (and the caller's id / count / byte-map arrays,
    // which CTA 0 writes) may still be in use by the kernel before this one: wait first.
    pdl_wait();
    if (tid == 0) BAS_TRACE_SET(19, BAS_TRACE_CLOCK() - hdr->t0);   // previous kernel done
    const int kept = fused_select(p, s_stage, s_ids, hdr->sel_warp_cnt, &hdr->sel_keep, rank, C, tid, kUmmaThreads,
                                  hdr->t0);
    if (tid == 0) hdr->k_act = kept;
    __syncthreads();
  }

  int k_act = 0;
  // Row-parallel sum over ranks (epilogue threads only): this call's sequence number in the
  // exchange area and the partial buffer it selects.
  unsigned int tp_epoch = 0;
  size_t tp_slot = 0;       // word offset, inside any rank's area, of this rank's array in the current receive buffer
  auto tp_send = [&](int row, int col, float v) { tp_send_word(p.tp, tp_epoch, tp_slot, row, col, v); };
  int armed_next = warp, armed_cnt = 0;   // producer warps: next group to arm, groups armed so far

  const int P = p.issuers;
  if (warp < kProducers) {
    // ------------------------------ id staging (warp 0) + producers ------------------------------
    if (warp == 0) {
      if (SEL) {
        k_act = hdr->k_act;     // the list is already in s_ids
      } else {
        if (!early_ids) pdl_wait();
        k_act = warp_stage_ids(p.ids, p.count_dev, p.k_host, p.bitmap, p.nb, s_ids, p.status, lane, early_ids,
                               first_ids);
      }
      if (lane == 0) {
        hdr->k_act = k_act;
        mbar_arrive(&hdr->ids_ready);
        BAS_TRACE_SET(9, BAS_TRACE_CLOCK() - hdr->t0);    // id list staged
      }
      pdl_launch_dependents();
    } else {
      // ordered after warp 0's wait for the previous kernel by the barrier
      if (__all_sync(0xffffffffu, mbar_wait_for(&hdr->ids_ready, 0, abort_flag, p.wait_cycles))) k_act = hdr->k_act;
    }
    const int k_mine = (k_act > rank) ? (k_act - rank + C - 1) / C : 0;
    const int M = n_sub * k_mine;                // tiles of this CTA: sub-tile major, active block minor
    const int NG = (M + G - 1) / G;              // groups = barrier hand-offs
    if (M > 0 && warp < P) {
      // One pass per ring group; producer warp w takes groups w, w+P, ...  Lane l owns tile l of
      // the group: it works out that tile's addresses (the integer divisions run side by side in the
      // lanes), the byte counts are added across the warp, lane 0 waits for the slot and arms its
      // barrier, then every lane issues its own two copies.  Slot index and lap are carried along.
      auto lane_tile = [&](int g, int& sub, int& j, int& wbytes) -> bool {
        const int m = g * G + lane;
        if (lane >= G || m >= M) return false;
        sub = (n_sub == 1) ? 0 : m / k_mine;
        j = s_ids[rank + (m - sub * k_mine) * C];
        wbytes = min(TW, width - sub * TW) * kRowBytes;
        return true;
      };
      // The activations are re-read by every CTA and by the next call: evict-last.  The weights take
      // the default policy: marked evict-first they ran 6-17 % slower where a caller replays one call
      // on one weight that fits in L2 (the reference's own timing protocol), and no faster cold.
      const uint64_t pol_x = l2_policy_evict_last();
      int g = warp;
      if (early_ids && !early_x) {
        // Stream the first ring-full of weight chunks while the previous kernel is still draining,
        // then wait for it before loading X.
        const int ahead = min(S, NG);
        for (int ga = warp; ga < ahead; ga += P) {
          int sub = 0, j = 0, wbytes = 0;
          const bool have = lane_tile(ga, sub, j, wbytes);
          const int total = __reduce_add_sync(0xffffffffu, have ? wbytes + kXTileBytes : 0);
          if (lane == 0) mbar_arrive_expect_tx(&hdr->full[ga], total);
          __syncwarp();
          if (have)
            bulk_copy_g2s(s_stage + (size_t)ga * stage_bytes + (size_t)lane * tile_bytes,
                          p.packed + ((size_t)j * p.npad + n0 + sub * TW) * kRowBytes, wbytes, &hdr->full[ga]);
          armed_next = ga + P;
          ++armed_cnt;
        }
        pdl_wait();
        for (int ga = warp; ga < ahead; ga += P) {
          int sub = 0, j = 0, wbytes = 0;
          if (lane_tile(ga, sub, j, wbytes))
            tma_load_2d_hint(s_stage + (size_t)ga * stage_bytes + (size_t)lane * tile_bytes + p.wslot, &xmap, j * kBlockK,
                             0, &hdr->full[ga], pol_x);
        }
        g = armed_next;
      }
      int s = g % S, lap = g / S;   // slot of group g and how often the slot has been used before
      for (; g < NG; g += P) {
        [[maybe_unused]] const long long tr0 = BAS_TRACE_CLOCK();
        int sub = 0, j = 0, wbytes = 0;
        const bool have = lane_tile(g, sub, j, wbytes);
        const int total = __reduce_add_sync(0xffffffffu, have ? wbytes + kXTileBytes : 0);
        bool ok = true;
        if (lane == 0) {
          if (lap > 0) ok = mbar_wait_for(&hdr->empty[s], (lap - 1) & 1, abort_flag, p.wait_cycles);
          if (ok) mbar_arrive_expect_tx(&hdr->full[s], total);
        }
        if (!__shfl_sync(0xffffffffu, ok, 0)) {
          if (lane == 0) {
            atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
            hdr->abort_flag = 1;
          }
          break;
        }
        [[maybe_unused]] const long long tr1 = BAS_TRACE_CLOCK();
        if (have) {
          uint8_t* st = s_stage + (size_t)s * stage_bytes + (size_t)lane * tile_bytes;
          bulk_copy_g2s(st, p.packed + ((size_t)j * p.npad + n0 + sub * TW) * kRowBytes, wbytes, &hdr->full[s]);
          tma_load_2d_hint(st + p.wslot, &xmap, j * kBlockK, 0, &hdr->full[s], pol_x);
        }
        armed_next = g + P;
        ++armed_cnt;
        if (lane == 0) {
          BAS_TRACE_SET(64 + g, tr1 - hdr->t0);                     // slot free seen by the producer
          BAS_TRACE_SET(128 + g, BAS_TRACE_CLOCK() - hdr->t0);      // group's copies issued
          BAS_TRACE_ADD(0, tr1 - tr0);                              // producer: waiting for a free slot
          BAS_TRACE_ADD(1, BAS_TRACE_CLOCK() - tr1);                // producer: issuing a slot's copies
          BAS_TRACE_ADD(2, 1);
        }
        s += P;
        while (s >= S) {
          s -= S;
          ++lap;
        }
      }
    }
  } else {
    bool ok = __all_sync(0xffffffffu, mbar_wait_for(&hdr->ids_ready, 0, abort_flag, p.wait_cycles));
    k_act = hdr->k_act;
    const int k_mine = (ok && k_act > rank) ? (k_act - rank + C - 1) / C : 0;
    const int M = n_sub * k_mine;

    if (warp < kEpiWarp0) {
      // ------------------------------ MMA issuers (one thread per warp) ------------------------------
      // Issuing one tcgen05.mma costs its thread on the order of a hundred cycles, far more than the
      // tensor core needs for a 128 x Bpad x 16 product.  Up to four warps therefore issue side by
      // side, each into an accumulator of its own; the epilogue adds them in issuer order.
      const int w = warp - kProducers;
      const int NI = P;
      if (lane == 0 && ok && w < NI && M > 0) {
        // Ring group g belongs to issuer g % NI alone: it waits for the group, multiplies its tiles
        // and frees the slot, so a hand-off costs one wait and one commit per group, not one per
        // issuer.  The assignment is a function of the shape only, hence so is the summation order.
        const uint32_t d = tmem_base + (uint32_t)(w * 64);   // this issuer's accumulator
        const int NG = (M + G - 1) / G;
        int cur_sub = 0;       // sub-tile this issuer's accumulator currently holds
        bool fresh = true;     // nothing multiplied into it yet
        // Passes with accumulator columns of their own (pass s at column offset s * BPAD): nothing is
        // handed to the epilogue between passes, so a CTA whose epilogue may not store yet (it waits for
        // the preceding kernel) keeps multiplying; one hand-over at the very end.
        const bool multi = (p.flags & kFlagMultiAcc) != 0;
        bool any_mma = false;
        // Finish with sub-tiles [cur_sub, target): tell the epilogue (the commit waits for this
        // issuer's MMAs), then wait until it has drained them before the accumulator is reused.
        auto advance_to = [&](int target) -> bool {
          while (cur_sub < target) {
            if (multi && cur_sub + 1 < n_sub) {
              ++cur_sub;
              fresh = true;
              continue;
            }
            if (w == 0) BAS_TRACE_SET(16, BAS_TRACE_CLOCK() - hdr->t0);   // issuer 0: last MMA of the sub-tile issued
            if (multi ? any_mma : !fresh) umma_commit(&hdr->acc_full);
            else mbar_arrive(&hdr->acc_full);
            if (!multi && cur_sub + 1 < n_sub && !mbar_wait_for(&hdr->acc_empty, cur_sub & 1, abort_flag, p.wait_cycles)) return false;
            ++cur_sub;
            fresh = true;
          }
          return true;
        };
        int s = w % S, fph = (w / S) & 1;
        for (int g = w; g < NG && ok; g += NI) {
          [[maybe_unused]] const long long tr0 = BAS_TRACE_CLOCK();
          if (!mbar_wait_for(&hdr->full[s], fph, abort_flag, p.wait_cycles)) {
            ok = false;
            break;
          }
          if (g == 0) BAS_TRACE_SET(15, BAS_TRACE_CLOCK() - hdr->t0);   // first group landed
          [[maybe_unused]] const long long tr1 = BAS_TRACE_CLOCK();
          tc_fence_after_sync();
          int m = g * G;
          int sub = (n_sub == 1) ? 0 : m / k_mine;
          int ii = m - sub * k_mine;
          for (int pos = 0; pos < G && m < M; ++pos, ++m) {
            if (sub != cur_sub && !advance_to(sub)) {
              ok = false;
              break;
            }
            const uint32_t st = smem_u32(s_stage + (size_t)s * stage_bytes + (size_t)pos * tile_bytes);
            const uint64_t bdesc = umma_desc_kmajor_sw128(st + p.wslot);
            const uint64_t adesc = umma_desc_kmajor_sw128(st);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              // 16 channels = 32 bytes along K: +2 in the descriptor's 16-byte address units; the
              // first MMA into a fresh accumulator overwrites it instead of adding
              umma_f16_ss(d + (multi ? (uint32_t)(cur_sub * BPAD) : 0u), adesc + (uint64_t)(2 * ks),
                          bdesc + (uint64_t)(2 * ks), kIdesc, (fresh && ks == 0) ? 0u : 1u);
            }
            fresh = false;
            any_mma = true;
            if (++ii == k_mine) {
              ii = 0;
              ++sub;
            }
          }
          if (!ok) break;
          umma_commit(&hdr->empty[s]);   // the slot is free once these MMAs have read it
          if (w == 0) {
            BAS_TRACE_ADD(4, tr1 - tr0);                    // issuer 0: waiting for data
            BAS_TRACE_ADD(5, BAS_TRACE_CLOCK() - tr1);      // issuer 0: issuing a group's MMAs
            BAS_TRACE_ADD(6, 1);
          }
          s += NI;
          while (s >= S) {
            s -= S;
            fph ^= 1;
          }
          // nothing more of the current sub-tile in this issuer's next group: let the epilogue have
          // it now rather than when that group has landed
          if (n_sub > 1 && (g + NI) * G < M) {
            const int sub2 = ((g + NI) * G) / k_mine;
            if (sub2 > cur_sub) ok = advance_to(sub2);
          }
        }
        if (ok) ok = advance_to(n_sub);
        if (!ok) {
          atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
          hdr->abort_flag = 1;
        }
      }
    } else {
      // ---------------- epilogue: two sets of 4 warps, one TMEM lane quarter per warp ----------------
      // Both sets see the same 128 accumulator rows (output columns); they divide the batch columns
      // in chunks of 16 (a batch of up to 16 rows is one chunk: the second set then idles).
      const int q = warp & 3;               // a warp may only read TMEM lanes [32*(warp%4), +32)
      const int r = q * 32 + lane;          // row of the sub-tile = output column n0 + 128*sub + r
      const int et = tid - 32 * kEpiWarp0;  // 0..255
      const int eset = et >> 7;             // 0 or 1
      constexpr int kChunks = BPAD / 16;
      constexpr int kChunks0 = (kChunks + 1) / 2;   // set 0's chunks; set 1 takes the rest
      if (early_ids && !late_wait) pdl_wait();   // before the first write to Y (late_wait: at the stores)
      const bool multi = (p.flags & kFlagMultiAcc) != 0;   // see the issuers: one hand-over for all passes
      if (TP) {
        // The rank's call counter: advanced by the last CTA to finish the previous call, i.e. before
        // the wait above (or warp 0's, which the id barrier orders before this point) returned.
        tp_epoch = __ldcg((const unsigned int*)p.tp.own) + 1u;
        tp_slot = (size_t)kTpHeaderBytes / 8 +
                  ((size_t)(tp_epoch & 1u) * (size_t)p.tp.world + (size_t)p.tp.rank) * (size_t)p.tp.src_words;
      }

      if (TP && ok && k_act == 0) {
        // empty active set on this rank: its partial of the elements this CTA owns is zero
        const int rz = et & 127;
        for (int c0 = 0; c0 < width; c0 += kTileN)
          if (c0 + rz < width && n0 + c0 + rz < p.n)
            for (int row = rank + C * eset; row < p.batch; row += 2 * C) tp_send(row, n0 + c0 + rz, 0.f);
      } else if (ok && k_act == 0) {
        // empty active set: the epilogue threads of the whole grid zero Y between them
        if (late_wait) pdl_wait();
        const long long total = (long long)p.batch * p.n;
        for (long long e = (long long)blockIdx.x * kEpiThreads + et; e < total; e += (long long)gridDim.x * kEpiThreads)
          p.y[(e / p.n) * p.ldy + (e % p.n)] = __float2half_rn(0.f);   // +0 in either format
      } else if (ok) {
        for (int sub = 0; sub < n_sub && ok; ++sub) {
          const int wsub = min(TW, width - sub * TW);
          if (k_mine > 0 && (!multi || sub == 0)) {
            // warp-uniform verdict: tcgen05.ld below needs the whole warp
            if (!__all_sync(0xffffffffu, mbar_wait_for(&hdr->acc_full, multi ? 0 : (sub & 1), abort_flag, p.wait_cycles))) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (et == 0) BAS_TRACE_SET(10, BAS_TRACE_CLOCK() - hdr->t0);   // accumulators final
          }
          // issuer w holds a partial of this sub-tile iff one of the ring groups w, w + P, ...
          // contains one of its tiles
          const int g_lo = (k_mine > 0) ? (sub * k_mine) / G : 0;
          const int g_hi = (k_mine > 0) ? ((sub + 1) * k_mine - 1) / G : -1;

          // Batch columns [16*CH0, 16*(CH0+NCH)): read the issuers' accumulators (as many
          // per tcgen05.wait as the registers allow), add them in issuer order, then store the
          // values (no cluster) or push them to the CTAs that own the rows.
          auto emit = [&](auto ch0_c, auto nch_c) {
            constexpr int CH0 = decltype(ch0_c)::value, NCH = decltype(nch_c)::value;
            constexpr int NV = NCH * 16;
            constexpr int IB = (BPAD == 16) ? 4 : (NCH == 1) ? 2 : 1;   // issuers read per wait (register budget: 128 per thread)
            float v[NV];
#pragma unroll
            for (int b = 0; b < NV; ++b) v[b] = 0.f;
            if (k_mine > 0) {
#pragma unroll
              for (int w0 = 0; w0 < kIssuers; w0 += IB) {
                if (w0 < P) {   // warp-uniform
                  uint32_t regs[IB][NCH][16];
#pragma unroll
                  for (int wi = 0; wi < IB; ++wi)
                    if (w0 + wi < P) {
#pragma unroll
                      for (int cc = 0; cc < NCH; ++cc)
                        tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) +
                                               (uint32_t)((w0 + wi) * 64 + (CH0 + cc) * 16 + (multi ? sub * BPAD : 0)),
                                           regs[wi][cc]);
                    }
                  tmem_ld_wait();
#pragma unroll
                  for (int wi = 0; wi < IB; ++wi) {
                    const int w = w0 + wi;
                    if (w < P && (w - g_lo % P + P) % P <= g_hi - g_lo) {   // issuer order: the sum never depends on timing
#pragma unroll
                      for (int cc = 0; cc < NCH; ++cc)
#pragma unroll
                        for (int e = 0; e < 16; ++e) v[cc * 16 + e] += __uint_as_float(regs[wi][cc][e]);
                    }
                  }
                }
              }
            }
            if (et == 0) BAS_TRACE_SET(18, BAS_TRACE_CLOCK() - hdr->t0);   // accumulators read and added
            const int rr = r;   // column within the pass
            if (C == 1) {
              if (late_wait) pdl_wait();   // returns at once from the second pass on
              const int col = n0 + sub * TW + rr;
              if (rr < wsub && col < p.n) {
                if (TP) {
#pragma unroll
                  for (int b = 0; b < NV; ++b)
                    if (16 * CH0 + b < p.batch) tp_send(16 * CH0 + b, col, v[b]);
                } else {
#pragma unroll
                  for (int b = 0; b < NV; ++b)
                    if (16 * CH0 + b < p.batch) store_out16(p.y + (size_t)(16 * CH0 + b) * p.ldy + col, v[b], bf16);
                }
              }
            } else {
              // Cluster mode (one pass per CTA): batch row b is finished by rank b % C.  Push this
              // CTA's partial of each row into the owner's shared memory; the stores are posted, the
              // cluster barrier below makes them visible.
              // Layout of the receive buffer: [source rank][column r][row slot], slots contiguous,
              // so that four of a thread's values for one owner go out as one 16-byte store.
              // Within a column the four-slot groups are XOR-swizzled by the column index, so that
              // neither these 16-byte stores nor the owner's 16-byte loads pile up on a few banks.
              const int nbi = BPAD / C;        // row slots per (source rank, column); a multiple of 4
              const int sw = red_swizzle(nbi, r);
              float* mine_l = s_red + (rank * kTileN + r) * nbi;
              const uint32_t mine = smem_u32(mine_l);
              uint32_t owner[4];
#pragma unroll
              for (int o = 0; o < 4; ++o) owner[o] = dsmem_addr(mine, (uint32_t)(o & (C - 1)));
              if (C == 4) {
#pragma unroll
                for (int o = 0; o < 4; ++o)
#pragma unroll
                  for (int c4 = 0; c4 < NCH; ++c4) {   // slots 4*b4 .. 4*b4+3 <-> rows 16*b4 + o + {0,4,8,12}
                    const int b4 = CH0 + c4;
                    if (16 * b4 + o < p.batch) {
                      const float4 val = make_float4(v[16 * c4 + o], v[16 * c4 + o + 4], v[16 * c4 + o + 8],
                                                     v[16 * c4 + o + 12]);
                      if (o == rank) *(float4*)(mine_l + 4 * (b4 ^ sw)) = val;   // own rows stay local
                      else dsmem_st_v4_f32(owner[o] + (uint32_t)(16 * (b4 ^ sw)), val.x, val.y, val.z, val.w);
                    }
                  }
              } else {
#pragma unroll
                for (int o = 0; o < 2; ++o)
#pragma unroll
                  for (int c8 = 0; c8 < 2 * NCH; ++c8) {   // slots 4*b8 .. 4*b8+3 <-> rows 8*b8 + o + {0,2,4,6}
                    const int b8 = 2 * CH0 + c8;
                    if (8 * b8 + o < p.batch) {
                      const float4 val = make_float4(v[8 * c8 + o], v[8 * c8 + o + 2], v[8 * c8 + o + 4],
                                                     v[8 * c8 + o + 6]);
                      if (o == rank) *(float4*)(mine_l + 4 * (b8 ^ sw)) = val;   // own rows stay local
                      else dsmem_st_v4_f32(owner[o] + (uint32_t)(16 * (b8 ^ sw)), val.x, val.y, val.z, val.w);
                    }
                  }
              }
            }
          };
          using std::integral_constant;
          if constexpr (kChunks == 1) {
            if (eset == 0) emit(integral_constant<int, 0>{}, integral_constant<int, 1>{});
          } else {
            if (eset == 0) emit(integral_constant<int, 0>{}, integral_constant<int, kChunks0>{});
            else emit(integral_constant<int, kChunks0>{}, integral_constant<int, kChunks - kChunks0>{});
          }
          if (et == 0) BAS_TRACE_SET(17, BAS_TRACE_CLOCK() - hdr->t0);   // accumulators drained and stored / pushed
          if (k_mine > 0) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&hdr->acc_empty);
          }
        }
      }
      if (!ok) {
        atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
        hdr->abort_flag = 1;
      }
    }
  }

  // A warp of which single lanes ran a role above must be whole again before it joins a CTA-wide
  // barrier: an arrival counts for 32 threads however many lanes make it.
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0) BAS_TRACE_SET(11, BAS_TRACE_CLOCK() - hdr->t0);    // roles done
  if (C > 1) {
    // Every CTA of the cluster has pushed its partials once all have passed this barrier; rank i
    // then adds, in rank order, what it received for batch rows i, i+C, ... and stores them.  Nothing
    // touches a peer's shared memory after the barrier, so CTAs may leave independently.
    cluster_sync_all();
    if (hdr->k_act > 0 && hdr->abort_flag == 0 && warp >= kEpiWarp0) {
      if (late_wait) pdl_wait();
      const int r = (tid - 32 * kEpiWarp0) & 127, eset = (tid - 32 * kEpiWarp0) >> 7;
      const int nbi = BPAD / C;
      const int sw = red_swizzle(nbi, r);
      {
        const int rr = r, col = n0 + rr;
        if (rr < width && col < p.n) {
          const float* half_red = s_red;
          // slot t of this rank is batch row t * C + rank; four slots per 16-byte load
          for (int qd = eset; 4 * qd * C + rank < p.batch; qd += 2) {   // the two warp sets alternate
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (q < C) {
                const float4 t = *(const float4*)(half_red + (q * kTileN + r) * nbi + 4 * (qd ^ sw));
                sum.x += t.x;
                sum.y += t.y;
                sum.z += t.z;
                sum.w += t.w;
              }
            const int row0 = 4 * qd * C + rank;
            const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (row0 + e * C < p.batch) {
                if (TP) tp_send(row0 + e * C, col, vals[e]);
                else store_out16(p.y + (size_t)(row0 + e * C) * p.ldy + col, vals[e], bf16);
              }
          }
        }
      }
    }
  }
  if (TP && warp >= kEpiWarp0) {
    // ---- sum over the ranks of the box ----
    // CTA c of every rank produces the same rows and columns of its rank's partial and has sent them
    // to all ranks.  Collect: poll (bounded) this rank's own receive buffer until the word of every
    // source rank carries this call's number, add the partials in rank order and store Y.  A peer
    // can be at most one call ahead of this rank, and it writes the other buffer then.
    const int et = tid - 32 * kEpiWarp0, eset = et >> 7, rz = et & 127;
    const unsigned long long* recv = (const unsigned long long*)p.tp.own + (size_t)kTpHeaderBytes / 8 +
                                     (size_t)(tp_epoch & 1u) * (size_t)p.tp.world * (size_t)p.tp.src_words;
    const long long t_start = clock64();
    bool good = hdr->abort_flag == 0;
    for (int c0 = 0; c0 < width && good; c0 += kTileN) {
      const int col = n0 + c0 + rz;
      if (c0 + rz < width && col < p.n)
        for (int row = rank + C * eset; row < p.batch && good; row += 4 * C) {
          // two of this thread's rows per round, all their source words requested together: the
          // round trips to memory overlap instead of adding up
          const int row2 = row + 2 * C;
          const bool have2 = row2 < p.batch;
          const size_t off = (size_t)row * (size_t)p.tp.ldp + (size_t)col;
          const size_t off2 = (size_t)(have2 ? row2 : row) * (size_t)p.tp.ldp + (size_t)col;
          unsigned long long words[kTpMaxRanks], words2[kTpMaxRanks];
#pragma unroll
          for (int q = 0; q < kTpMaxRanks; ++q) {
            words[q] = (q < p.tp.world) ? ld_relaxed_sys_u64(recv + (size_t)q * (size_t)p.tp.src_words + off) : 0ull;
            words2[q] = (q < p.tp.world) ? ld_relaxed_sys_u64(recv + (size_t)q * (size_t)p.tp.src_words + off2) : 0ull;
          }
          float sum = 0.f, sum2 = 0.f;
#pragma unroll
          for (int q = 0; q < kTpMaxRanks; ++q)
            if (q < p.tp.world) {   // rank order
              while ((unsigned int)(words[q] >> 32) != tp_epoch || (unsigned int)(words2[q] >> 32) != tp_epoch) {
                if (clock64() - t_start > p.wait_cycles) {
                  good = false;
                  break;
                }
                __nanosleep(32);
                words[q] = ld_relaxed_sys_u64(recv + (size_t)q * (size_t)p.tp.src_words + off);
                words2[q] = ld_relaxed_sys_u64(recv + (size_t)q * (size_t)p.tp.src_words + off2);
              }
              sum += __uint_as_float((unsigned int)words[q]);
              sum2 += __uint_as_float((unsigned int)words2[q]);
            }
          if (good) {
            store_out16(p.y + (size_t)row * p.ldy + col, sum, bf16);
            if (have2) store_out16(p.y + (size_t)row2 * p.ldy + col, sum2, bf16);
          }
        }
    }
    if (!good && hdr->abort_flag == 0) atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
    // The rank's call counter advances whatever happened, so that the ranks stay in step: the last CTA
    // to get here does it (every CTA has read the counter by then; the next call reads it only after
    // this grid has completed).
    if (et == 0) {
      unsigned int* ctr = (unsigned int*)p.tp.own;
      __threadfence();
      if (atomicAdd(ctr + 1, 1u) == gridDim.x - 1) {
        ctr[1] = 0u;
        ctr[0] = tp_epoch;
        __threadfence();
      }
    }
  }
  if (tid == 32 * kEpiWarp0) BAS_TRACE_SET(12, BAS_TRACE_CLOCK() - hdr->t0);    // cluster combine done
  if (hdr->abort_flag != 0 && warp < P && lane == 0) {
    // Gave up somewhere: do not leave while copies may still be landing in this CTA's memory.
    int zero = 0;
    const int per_lap = S / P;   // this warp's groups in one trip round the ring
    for (int i = 0, g = armed_next - P; i < min(armed_cnt, per_lap) && g >= 0; ++i, g -= P)
      (void)mbar_wait_for(&hdr->full[g % S], (g / S) & 1, &zero, p.wait_cycles);
  }
  if (warp == kEpiWarp0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  BAS_TRACE_LAUNCH_END();
}

// ---------------------------------------------------------------------------------------------
// host side: tensor maps for X, the work split and the launch
// ---------------------------------------------------------------------------------------------
struct MapKey {
  const void* x;
  long long ldx;
  int batch, k, bpad, bf16;
  bool operator==(const MapKey& o) const {
    return x == o.x && ldx == o.ldx && batch == o.batch && k == o.k && bpad == o.bpad && bf16 == o.bf16;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& m) const {
    size_t h = (size_t)m.x;
    h = h * 1000003u ^ (size_t)m.ldx;
    h = h * 1000003u ^ (size_t)m.batch;
    h = h * 1000003u ^ (size_t)m.k;
    return h * 1000003u ^ (size_t)(m.bpad * 2 + m.bf16);
  }
};

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = (PFN_cuTensorMapEncodeTiled_v12000)ptr;
    }
  });
  return fn;
}

// X[batch, K] fp16 or bf16, row stride ldx: inner dimension K, box {64 channels, bpad rows}, 128-byte swizzle.
cudaError_t get_x_tensor_map(const GemmParams& p, int bpad, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const int bf16 = (p.flags & kFlagBf16) != 0 ? 1 : 0;
  const MapKey key{p.x, p.ldx, p.batch, p.k, bpad, bf16};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return cudaSuccess;
    }
  }
  PFN_cuTensorMapEncodeTiled_v12000 encode = get_encode_fn();
  if (encode == nullptr) return cudaErrorNotSupported;
  const cuuint64_t gdim[2] = {(cuuint64_t)p.k, (cuuint64_t)p.batch};
  const cuuint64_t gstride[1] = {(cuuint64_t)p.ldx * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)bpad};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(p.x), gdim, gstride, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
  }
  return cudaSuccess;
}

constexpr size_t kSmemBudget = 224 * 1024;

// How many clusters of `cluster` CTAs of this kernel the device can hold at once (cached).
template <int BPAD>
int max_resident_clusters(int cluster, size_t smem, int sm_count) {
  static std::mutex mu;
  static std::unordered_map<long long, int> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  const long long key = ((long long)dev << 40) ^ ((long long)cluster << 32) ^ (long long)smem;
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sm_count / cluster * cluster));
  cfg.blockDim = dim3(kUmmaThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, umma_colsplit_kernel<BPAD, false, false>, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  std::lock_guard<std::mutex> lk(mu);
  cache[key] = n;
  return n;
}

template <int BPAD>
cudaError_t launch_umma_b(GemmParams p, int sm_count, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(umma_colsplit_kernel<BPAD, false, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(umma_colsplit_kernel<BPAD, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               227 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(umma_colsplit_kernel<BPAD, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  const int units = p.npad / 8;
  const size_t fixed = umma_fixed_smem(p.nb);

  // Work split (measured over output widths 512..22016, 1.5..65 MB of active weights, batches 2..64).
  // Two things decide it.  (1) How many CTAs: consecutive calls of a stream overlap - the next call's
  // CTAs come up on free SMs, stage their ids and stream a ring-full of weights while this call is
  // still running - but only if this call leaves SMs free; and one SM takes in about 100 GB/s, so
  // about half the SMs already saturate HBM.  Hence: about 96 KiB of active weights per CTA for
  // small problems, at most half the SMs up to about 25 MB, all but twenty of them beyond.  (2) The
  // shape: a cluster of 4 CTAs per column range of up to 128 columns (the cluster splits the active
  // blocks, quartering the copies and MMAs issued per byte and the activation traffic per SM, and
  // finishes its range in one pass), else a cluster of 2, else one CTA per range walking 128-column
  // passes; the first of these whose CTA count stays within 15 % of the target is taken.
  const int forced = (p.flags >> 8) & 7;
  const int cta_cap = ((p.flags >> 16) & 0xff) != 0 ? ((p.flags >> 16) & 0xff) : sm_count;   // tuning knob
  // active blocks expected: the list length, or with a byte map the caller's hint (else half of all)
  const int k_est = p.k_host > 0 ? p.k_host : (p.nb + 1) / 2;
  const double bytes = (double)k_est * kBlockK * 2.0 * (double)p.n;
  int target = (int)(bytes / (96.0 * 1024.0)) + 1;
  if (target < 16) target = 16;
  if (target > sm_count / 2) target = (bytes >= 25.0e6) ? sm_count - 20 : sm_count / 2;
  // a call that also exchanges its result with the other ranks of a box spreads that work (a few
  // words per thread to send and to wait for) over at least half the SMs
  if (p.tp.world > 1 && target < sm_count / 2) target = sm_count / 2;
  if (target > cta_cap) target = cta_cap;
  const int r_min = (units + kTileN / 8 - 1) / (kTileN / 8);   // fewest ranges of at most 128 columns
  // without a cluster: one pass per CTA (a second pass re-reads X) if that takes at most twice the
  // target number of CTAs
  int cluster = 1, ranges = (r_min > target && r_min <= 2 * target && r_min <= cta_cap) ? r_min : target;
  if (ranges > units) ranges = units;
  for (int c = 4; c >= 2 && forced != 1; c -= 2) {
    if (forced != 0 && c != forced) continue;
    int resident = max_resident_clusters<BPAD>(c, kSmemBudget, sm_count);
    if (resident > cta_cap / c) resident = cta_cap / c;
    if (resident > units) resident = units;
    if (r_min > resident) continue;                               // the widest range must fit one pass
    int r = target / c;
    if (r < r_min) r = r_min;
    if (r > resident) r = resident;
    if (forced == 0 && 20 * r * c > 23 * target) continue;        // too many CTAs for the work
    cluster = c;
    ranges = r;
    break;
  }
  // A call that declared both its id list and X stable does not depend on the call before it until
  // it stores: such calls pipeline several deep (each waits, in its epilogue, for its predecessor to
  // complete, so the stores stay in stream order).  Small grids are then best - one CTA per
  // 128-column range, no cluster, nothing to combine - because the next calls fill the other SMs
  // (measured: 32 CTAs per call for 4096 columns, 86 for 11008).
  const bool pipelined = (p.flags & kFlagStableX) != 0 && (p.flags & kFlagStableIds) != 0 && p.count_dev == nullptr &&
                         p.sel.mode == 0 && p.tp.world == 0;
  if (pipelined && forced == 0 && ((p.flags >> 16) & 0xff) == 0 && r_min >= 16 && r_min <= sm_count) {
    cluster = 1;
    ranges = r_min;
    // Wide outputs (more ranges than half the SMs) at batches of up to 32 rows, where the caller says
    // that the call after this one is independent too (BAS_GEMM_NEXT_INDEPENDENT: a deep chain): two
    // 128-column passes per CTA, each pass with accumulator columns of its own, so that again several
    // calls fit.  Followed by a call that has to wait for it, this grid is the slower one (measured on
    // the layer stack: up before down).
    if ((p.flags & kFlagNextIndependent) != 0 && r_min > sm_count / 2 && 2 * BPAD <= 64) {
      ranges = (r_min + 1) / 2;
      if (((units + ranges - 1) / ranges) * 8 <= 2 * kTileN) p.flags |= kFlagMultiAcc;
      else ranges = r_min;
    }
  }
  // Measured over the layer stack's shapes: waiting for the predecessor only at the stores pays (4-17 %)
  // when this call leaves at least half the SMs to its successors, and costs 7 % on the 86-CTA grid.
  if (pipelined && ranges * cluster <= sm_count / 2) p.flags |= kFlagLateWait;
  const int tile_cols = kTileN;
  const int wmax = ((units + ranges - 1) / ranges) * 8;
  const int wsub_max = wmax < tile_cols ? wmax : tile_cols;
  p.cluster = cluster;
  p.ranges = ranges;
  p.tile_cols = tile_cols;
  p.wslot = (wsub_max * kRowBytes + 1023) / 1024 * 1024;
  const size_t stage_bytes = (size_t)p.wslot + BPAD * 128;
  const size_t red_bytes = cluster > 1 ? (size_t)BPAD * kTileN * 4 : 0;   // partials pushed by the cluster
  // An MMA reads 128 rows (16 KiB) from the tile base whatever the tile's width: what the widest
  // tile does not cover itself is padding behind the ring.
  const size_t pad = (size_t)kMmaSpanBytes > (size_t)p.wslot ? (size_t)kMmaSpanBytes - (size_t)p.wslot : 0;
  if (fixed + red_bytes + pad + 2 * stage_bytes > kSmemBudget) return cudaErrorInvalidValue;
  const size_t room = kSmemBudget - fixed - red_bytes - pad;
  // One barrier hand-off costs a few hundred cycles per role: a slot gathers enough blocks (about
  // 24 KiB) for the hand-offs to stay off the critical path.
  int group = (int)((24 * 1024 + stage_bytes / 2) / stage_bytes);   // nearest
  if (group < 1) group = 1;
  if (group > 16) group = 16;
  int slots = (int)(room / (stage_bytes * group));
  if (slots < 4) {
    group = 1;
    slots = (int)(room / stage_bytes);
  }
  if (slots > kMaxStages) slots = kMaxStages;
  if (slots < 2) return cudaErrorInvalidValue;
  // Producer/issuer pairs: as many as possible while the ring (a multiple of the pair count) keeps
  // at least three quarters of the slots that fit; otherwise whatever keeps the most slots.
  int pairs = (p.flags >> 12) & 7;
  if (pairs < 2 || pairs > kIssuers || slots / pairs == 0) {
    pairs = 0;
    int best = 2;
    for (int c = kIssuers; c >= 2; --c) {
      const int kept = slots / c * c;
      if (kept * 4 >= slots * 3) {
        pairs = c;
        break;
      }
      if (kept > slots / best * best) best = c;
    }
    if (pairs == 0) pairs = best;
  }
  p.issuers = pairs;
  p.stages = slots / pairs * pairs;
  p.group = group;
  const size_t smem = fixed + red_bytes + pad + (size_t)p.stages * group * stage_bytes;

  CUtensorMap xmap;
  cudaError_t e = get_x_tensor_map(p, BPAD, &xmap);
  if (e != cudaSuccess) return e;
  if (p.sel.mode != 0) {
    // the in-kernel selection needs a cluster to share the scoring and room for its scratch in the ring
    // ... and pays only while a CTA's share of the scoring is small (every cluster repeats it:
    // measured against the two-launch chain, up to about 256 (block, row) pairs per CTA)
    const long long pairs_per_cta = (long long)((p.sel.nb_sel + cluster - 1) / cluster) * p.batch;
    const bool forced_sel = (p.flags & (1 << 24)) != 0;   // tuning knob: in-kernel selection whatever the size
    if (cluster < 2 || p.tp.world > 0 || (pairs_per_cta > 256 && !forced_sel) ||
        fused_select_scratch(p.sel.nb_sel, cluster, p.batch) > (size_t)p.stages * group * stage_bytes)
      return cudaErrorNotSupported;
    count_launch();
    return launch_with_pdl(umma_colsplit_kernel<BPAD, false, true>, ranges * cluster, kUmmaThreads, smem, cluster, stream,
                           p, xmap);
  }
  count_launch();
  if (p.tp.world > 0)
    return launch_with_pdl(umma_colsplit_kernel<BPAD, true, false>, ranges * cluster, kUmmaThreads, smem, cluster, stream,
                           p, xmap);
  return launch_with_pdl(umma_colsplit_kernel<BPAD, false, false>, ranges * cluster, kUmmaThreads, smem, cluster, stream, p,
                         xmap);
}

}  // namespace

// cuTensorMapEncodeTiled of the loaded driver (null if it has none); shared with the list kernel's host side.
void* tensor_map_encoder() { return (void*)get_encode_fn(); }

cudaError_t launch_umma(const GemmParams& p, int sm_count, cudaStream_t stream) {
  const int bpad = (p.batch + 15) / 16 * 16;
  switch (bpad) {
    case 16: return launch_umma_b<16>(p, sm_count, stream);
    case 32: return launch_umma_b<32>(p, sm_count, stream);
    case 48: return launch_umma_b<48>(p, sm_count, stream);
    case 64: return launch_umma_b<64>(p, sm_count, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace bas
