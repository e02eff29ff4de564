// A whole list of masked contractions as ONE persistent launch (bas_list_*).
//
// A decode step is a chain of small linears (224 for Llama-2-7B; the reference patches every one of
// them, scripts/bench_roundrobin_e2e_decode.py:331-503, and its benchmark sums them per step,
// scripts/bench_perstep_actual_kernel_speedup.py:268-293).  Launched one by one, each pays set-up,
// first-byte latency, accumulator read-out and the hand-over to the next kernel, during which its SMs
// do not stream.  Here the CTAs stay resident and walk the list:
//
//   * the ring of weight tiles runs across call boundaries: a call's weights never depend on the
//     call before it, so they are fetched while that call is still being finished;
//   * only a call's activation tiles wait - on a completion counter in global memory that the
//     CTAs finishing the call it depends on add to (release) and the reader polls (acquire, bounded);
//   * accumulators are double-buffered in tensor memory, so the MMAs of the next unit run while
//     the previous one is read out, combined across the cluster and stored.
//
// Work split: a cluster of C CTAs owns, for every call, one contiguous range of output columns
// (narrow outputs use fewer clusters, rotating, so that consecutive small calls land on different
// SMs); the range is walked in column tiles of at most 128; the cluster's CTAs deal the call's active
// blocks out round-robin and add their fp32 partials through distributed shared memory in rank
// order (mbarriers in the owner's shared memory, no cluster-wide barrier inside the loop).
//
// Roles per CTA: warps 0..3 issue copies (each compacts the call's id list for itself; warp 0 also
// publishes the call's tile counts to the other roles), warps 4..7 issue MMAs (one thread each, own
// accumulators), warps 8..15 read out, combine, store and signal completion.  Every wait is bounded
// by a launch parameter and reports through the status word.
#include "bas_kernels.cuh"

#include <cudaTypedefs.h>

#include <cstddef>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <new>
#include <type_traits>
#include <vector>

namespace bas {

namespace {

constexpr int kLProducers = 4;          // copy-issuing warps
constexpr int kLIssuers = 8;            // MMA-issuing warps available: issuing the four MMAs of a tile costs one thread
                                        // about 560 cycles (measured), the tensor core 92 to 156; eight threads keep it fed
constexpr int kLEpiWarp0 = kLProducers + kLIssuers;   // a multiple of 4: an epilogue warp reads the TMEM lane quarter warp % 4
constexpr int kLEpiThreads = 128;       // one epilogue warp per quarter
constexpr int kLThreads = 32 * kLEpiWarp0 + kLEpiThreads;
constexpr int kLMmaSpanBytes = 128 * kRowBytes;
// Every CTA reads every score of a selection entry at about the same time: one array would be one hot spot in the
// L2 (some six hundred warps on the same few lines).  The scoring warp writes each score to this many copies,
// in different lines, and a reading warp takes the copy that goes with its number.
constexpr int kSelReplicas = 16;
// Upper bits of the status word: the role of the first wait of a CTA that ran out (diagnosis only).
constexpr unsigned int kWhereCopyWarp = 0x100u, kWhereIssuer = 0x200u, kWhereEpilogue = 0x400u,
                       kWhereExchangeOwner = 0x800u, kWhereExchangeReader = 0x1000u;
// A wait that runs out leaves its role and its call index (bits 16-27) in the status word.  Of several, the one
// in the earliest call stays: later calls only wait for what that one did not deliver, but their waits may
// have started, and so run out, before it.  Roles of the same call are added together.
__device__ __forceinline__ void record_expiry(unsigned int* status, unsigned int where, int call) {
  const unsigned int c = (unsigned int)min(call, 4095);
  unsigned int old = *(volatile unsigned int*)status;
  for (;;) {
    const unsigned int old_call = (old >> 16) & 0xfffu;
    unsigned int want;
    if ((old & BAS_DEV_WAIT_EXPIRED) == 0u || c < old_call) want = (old & 0xffu) | BAS_DEV_WAIT_EXPIRED | where | (c << 16);
    else if (c == old_call) want = old | where;
    else return;
    if (want == old) return;
    const unsigned int seen = atomicCAS(status, old, want);
    if (seen == old) return;
    old = seen;
  }
}

// Device-side description of one call, written once by bas_list_create.
struct alignas(128) ListCallDev {
  CUtensorMap xmap;            // X[batch, K]: box {64 channels, BPAD rows}, 128-byte swizzle
  const uint8_t* packed;
  const int32_t* ids;
  const int32_t* count_dev;
  const uint8_t* bitmap;
  __half* y;
  long long ldy;
  int k_host, batch, n, nb;
  int units;                   // padded output columns / 8
  int ranges;                  // clusters that take part in this call
  int range_off;               // the first of them (the others follow, modulo the cluster count)
  int dep;                     // call whose completion X waits for, or -1
  unsigned int dep_contrib;    // CTAs that report the completion of call `dep`
  int tp_index;                // row-parallel calls: position among the list's exchanges (0, 1, ...); else -1
  // Selection inside the list.  A selection entry (n == 0) has no weights and no output; the copy warps of its
  // CTAs score the blocks of X, publish the scores, wait until all are there, and say for each of their blocks
  // whether it is among the kept ones.  It keeps, in the fields the copy warps hold in registers:
  //   packed = X, ids = its score array (see bas_list_create for the layout behind it), count_dev = {row stride
  //   of X in elements, reports the entry gets}, bitmap = {score kind, reports of the call it waits for};
  //   k_host = blocks to keep.
  // A contraction that takes its mask from entry e polls the entry's verdicts at its call boundary; it keeps:
  //   k_host = -(e + 1), ids = the entry's score array, count_dev = {the entry's blocks, unused},
  //   bitmap = {first block of the mask that is this call's block 0, unused}.
  int32_t* ids_out;            // such a contraction: where the kept ids of the whole mask go (ascending), or null
  // Output-block sparsity (bit 30 of range_off): the call computes only the 64-column blocks named in n_ids.  Its
  // column space is virtual - position q of the list is columns 64 q .. 64 q + 63, `units` counts those - and a
  // column tile is one block: the weights come from block n_ids[q] of the packed rows (w_rows per K block), the
  // results go to that block's columns of y or, `out_compact`, to the virtual ones.  Bit 29 of range_off: X holds
  // the active input blocks only, in list order (tile i reads columns 64 i .. 64 i + 63).
  const int32_t* n_ids;
  int w_rows;                  // padded output columns of the packed weight
  int out_compact;
  int pad[4];
};
constexpr int kRangeOffMask = 0xffff, kCall2d = 1 << 30, kCallXCompact = 1 << 29;
// Bit 28 of range_off.  A selection entry over a K-SHARDED activation (tensor-parallel lists): X holds this
// rank's blocks only (w_rows = their first block in the whole input, out_compact = the blocks of the whole
// input); the scores travel to every rank through the exchange area and a block's rank is taken among all of
// them.  A contraction that runs with such an entry's mask looks at the verdicts of its own blocks only.
constexpr int kCallSharded = 1 << 28;
constexpr unsigned int kStatusBadLayout = 0x40000000u;   // a descriptor field the kernel indexes with is out of range (never seen: the host checks)
static_assert(sizeof(ListCallDev) == 256, "call descriptor layout");

struct ListHeaderDev {
  unsigned int epoch;      // completed runs of the list: counters below are never reset, targets grow
  unsigned int arrived;    // CTAs of the current run that have finished
  unsigned int status;     // BAS_DEV_* bits
  unsigned int pad;
};

struct ListParams {
  const ListCallDev* calls;
  int n_calls;
  ListHeaderDev* hdr;
  unsigned int* done;        // [n_calls] completion counters
  int cluster;               // CTAs per cluster (1, 2, 4)
  int n_clusters;
  int stages;                // ring slots, a multiple of `pairs`
  int pairs;                 // copy warps in use (copy warp q issues the tiles t with t % pairs == q)
  int issuers;               // MMA-issuing warps in use, a multiple of `pairs` (issuer w multiplies the tiles t % issuers == w)
  int wslot;                 // bytes reserved per slot for a weight tile (multiple of 1024)
  int nb_max;                // largest K / 64 of the list
  int sel_nb_max;            // largest K / 64 of its selection entries (0: the list has none)
  int extended;              // the list has selection entries, output-block calls or compact X: the SEL variant runs it
  int sel_rep_stride;        // elements between the copies of an entry's score array (and of its verdict words)
  int bf16;
  int stall_call;            // tests of the expiry path: this call's dependency is never seen complete (-1: off)
  long long wait_cycles;     // bound of every wait
  TpExchange tp;             // lists with row-parallel calls: the group's exchange areas (world 0 = none)
  int n_tp_calls;            // exchanges per run
  int n_sharded;             // selection entries over sharded activations per run
#ifdef BAS_TRACE
  long long* trace;          // diagnostic build only
  int trace_cta;
#endif
};

struct ListSmemHeader {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t red_full[2];
  uint32_t tmem_base;
  int abort_flag;
  unsigned int calls_staged;   // records [0, calls_staged) are valid
  // Epilogue warps that have finished their part of a call.  One counter per call this CTA takes part in, four
  // in rotation: a warp can be two column tiles, so at most two such calls, ahead of the slowest one (the
  // accumulator buffers alternate), and its arrival for the later call must not be counted for the earlier.
  unsigned int epi_arrived[4];
  unsigned int dep_seen;       // 1 + the call whose completion copy warp 0 has seen last (0: none yet)
};

// Per-call record published by copy warp 0: bit 31 = this CTA takes part, bit 30 = its column tiles
// are at most 64 wide and multiplied with M = 64 instructions, bits 16..23 = column tiles of its
// range, bits 0..15 = active blocks of this CTA.
__device__ __forceinline__ unsigned int make_record(bool part, bool m64, int n_sub, int k_mine) {
  return (part ? 0x80000000u : 0u) | (m64 ? 0x40000000u : 0u) | ((unsigned int)n_sub << 16) | (unsigned int)k_mine;
}

// This cluster's share of a call.
struct Share {
  bool part;
  int n0, width, n_sub, tw;   // first column, columns, column tiles, columns per tile (multiple of 8)
};
__device__ __forceinline__ Share call_share(int units, int ranges, int range_off, int cid, int n_clusters) {
  Share s;
  int range = cid - (range_off & kRangeOffMask);
  if (range < 0) range += n_clusters;
  s.part = range < ranges;
  s.n0 = s.width = s.n_sub = 0;
  s.tw = 8;
  if (s.part && (range_off & kCall2d) != 0) {
    // output blocks: whole 64-column blocks per range, one block per column tile
    const int blocks = units >> 3;
    const int q0 = (int)((long long)range * blocks / ranges), q1 = (int)((long long)(range + 1) * blocks / ranges);
    s.n0 = q0 * 64;
    s.width = (q1 - q0) * 64;
    s.n_sub = q1 - q0;
    s.tw = 64;
  } else if (s.part) {
    s.n0 = col_begin(range, units, ranges);
    s.width = col_begin(range + 1, units, ranges) - s.n0;
    s.n_sub = (s.width + kTileN - 1) / kTileN;
    if (s.n_sub > 0) s.tw = ((s.width + s.n_sub - 1) / s.n_sub + 7) & ~7;
  }
  return s;
}

// Read-only load of a pointer-valued field of a call descriptor.
template <typename T>
__device__ __forceinline__ T* ldg_ptr(T* const* field) {
  return (T*)(uintptr_t)__ldg((const unsigned long long*)field);
}

// The fields of a call descriptor that the copy warps need, fetched as four 16-byte loads that stay
// where they are written (volatile), so that a call's descriptor can be requested two calls ahead
// and its id list one call ahead: at a call boundary everything is already in registers.
struct CallRegs {
  uint4 a, b, c, d;   // {packed, ids}, {count_dev, bitmap}, {k_host, batch, n, nb}, {units, ranges, range_off, dep}
};
__device__ __forceinline__ uint4 ld_nc_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}
__device__ __forceinline__ CallRegs load_call_regs(const ListCallDev* cd) {
  const uint8_t* base = (const uint8_t*)cd;
  CallRegs r;
  r.a = ld_nc_v4(base + offsetof(ListCallDev, packed));
  r.b = ld_nc_v4(base + offsetof(ListCallDev, count_dev));
  r.c = ld_nc_v4(base + offsetof(ListCallDev, k_host));
  r.d = ld_nc_v4(base + offsetof(ListCallDev, units));
  return r;
}
__device__ __forceinline__ const void* regs_ptr(unsigned int lo, unsigned int hi) {
  return (const void*)(uintptr_t)(((unsigned long long)hi << 32) | (unsigned long long)lo);
}

__device__ __forceinline__ int red_swizzle_l(int nbi, int r) {
  return nbi == 32 ? (r & 7) : nbi == 16 ? ((r >> 1) & 3) : nbi == 8 ? ((r >> 2) & 1) : 0;
}

// ---- selection inside the list ---------------------------------------------------------------
// Score of activation block j, by one warp: exactly the arithmetic of the selection kernel (bas_misc.cu), so
// that both give the same bits.  Eight lanes per (row, block) pair, 16 bytes per lane: exact squares summed in
// fp64 in element order, then over the eight lanes by a butterfly; optional square root; the rows added in
// row order; divided by the batch.  Rows go four at a time, sixteen in flight.  X may have been written by
// this launch: loads bypass the non-coherent path.  The result is the same in every lane.
__device__ __forceinline__ double warp_block_score(const __half* x, long long ldx, int batch, int j, bool bf16,
                                                   bool norm, int lane) {
  const int sub = lane & 7, grp = lane >> 3;
  double s = 0.0;
  for (int b0 = 0; b0 < batch; b0 += 16) {
    uint4 v[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int b = b0 + 4 * r + grp;
      v[r] = make_uint4(0u, 0u, 0u, 0u);
      if (b < batch) v[r] = __ldcg((const uint4*)(x + (size_t)b * (size_t)ldx + (size_t)j * kBlockK) + sub);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const unsigned int* wds = (const unsigned int*)&v[r];
      double e = 0.0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (bf16) {   // a bf16 is the upper half of an fp32; its square is taken in fp64 (range)
          const double lo = (double)__uint_as_float(wds[q] << 16), hi = (double)__uint_as_float(wds[q] & 0xffff0000u);
          e += lo * lo;
          e += hi * hi;
        } else {
          const float2 f = __half22float2(*(const __half2*)&wds[q]);
          e += (double)(f.x * f.x);   // a product of two fp16 values is exact in fp32
          e += (double)(f.y * f.y);
        }
      }
      e += __shfl_xor_sync(0xffffffffu, e, 1);
      e += __shfl_xor_sync(0xffffffffu, e, 2);
      e += __shfl_xor_sync(0xffffffffu, e, 4);
      if (norm) e = sqrt(e);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const double eg = __shfl_sync(0xffffffffu, e, 8 * g);
        if (b0 + 4 * r + g < batch) s += eg;
      }
    }
  }
  return s / (double)batch;
}

// TP: the variant for lists with row-parallel calls, whose epilogue exchanges partial sums with the other
// ranks of a box (a template parameter, so that the plain kernel carries none of that code).  SEL: the variant
// for lists with selection entries, output-block calls or compact activations, likewise.
template <int BPAD, bool TP, bool SEL>
__global__ void __launch_bounds__(kLThreads, 1) umma_list_kernel(const __grid_constant__ ListParams p) {
  constexpr int kXTileBytes = BPAD * 128;
  constexpr int kAccIssuers = (2 * kLIssuers * BPAD <= 512) ? kLIssuers : 4;   // tensor memory has 512 columns
  constexpr int kAccCols = 2 * kAccIssuers * BPAD;                    // two buffers of one accumulator per issuer
  constexpr int kTmemCols = kAccCols <= 128 ? 128 : kAccCols <= 256 ? 256 : 512;
  const uint32_t kFmt = p.bf16 ? ((1u << 7) | (1u << 10)) : 0u;
  const uint32_t kIdesc = umma_idesc_f16(128, BPAD) | kFmt, kIdesc64 = umma_idesc_f16(64, BPAD) | kFmt;
  const bool bf16 = p.bf16 != 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* sp = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  ListSmemHeader* hdr = (ListSmemHeader*)sp;
  sp += (sizeof(ListSmemHeader) + 127) / 128 * 128;
  unsigned int* s_rec = (unsigned int*)sp;                 // [n_calls]
  sp += ((size_t)p.n_calls * 4 + 127) / 128 * 128;
  uint16_t* s_ids_all = (uint16_t*)sp;                     // [kLProducers][nb_max]
  const size_t ids_stride = ((size_t)p.nb_max * 2 + 127) / 128 * 128;
  sp += ids_stride * kLProducers;
  uint2* s_def_all = (uint2*)sp;                           // [kLProducers][kMaxStages] deferred activation copies
  sp += sizeof(uint2) * kMaxStages * kLProducers;
  float* s_red = (float*)sp;                               // [2][source rank][128][row slots]
  const int C = p.cluster;
  if (C > 1) sp += 2 * (size_t)BPAD * kTileN * sizeof(float);
  uint8_t* s_stage = (uint8_t*)(((uintptr_t)sp + 1023) & ~(uintptr_t)1023);
  const int S = p.stages, P = p.pairs, PI = p.issuers;
  const int tile_bytes = p.wslot + kXTileBytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &hdr->abort_flag;
  const long long limit = p.wait_cycles;

  if (tid < S) {
    mbar_init(&hdr->full[tid], 1);
    mbar_init(&hdr->empty[tid], 1);
    fence_barrier_init();
  } else if (tid == 64) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&hdr->acc_full[b], PI);
      mbar_init(&hdr->acc_empty[b], kLEpiThreads / 32);
      mbar_init(&hdr->red_full[b], C * (kLEpiThreads / 32));
    }
    hdr->abort_flag = 0;
    hdr->calls_staged = 0u;
    for (int q = 0; q < 4; ++q) hdr->epi_arrived[q] = 0u;
    hdr->dep_seen = 0u;
    fence_barrier_init();
  }
  if (warp == kLEpiWarp0) {
    tmem_alloc(&hdr->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // peers arrive on this CTA's barriers: they must be initialised in every CTA before anyone starts
  if (C > 1) cluster_sync_all();
  const uint32_t tmem_base = hdr->tmem_base;

  // Everything read below (descriptors are fixed, but X, the id lists, the counters and the epoch)
  // may be written by the kernel before this one in the stream.
  pdl_wait();
  const unsigned int epoch = __ldcg(&p.hdr->epoch);
  // exchanges the group has completed before this run: exchange k of the list carries number tp_base + k + 1
  unsigned int tp_base = 0u, sel_base = 0u;
  if constexpr (TP) {
    tp_base = __ldcg((const unsigned int*)p.tp.own);
    sel_base = __ldcg((const unsigned int*)p.tp.own + 2);   // sharded selection entries completed before this run
  }

  const int rank = (C > 1) ? (int)cluster_ctarank() : 0;
  const int cid = blockIdx.x / C;
  int armed_cnt = 0;       // copy warps: tiles armed so far (lane 0)

  if (warp < kLProducers) {
    // ================================ copy warps ================================
    if (warp < P) {
      uint16_t* s_ids = (uint16_t*)((uint8_t*)s_ids_all + ids_stride * warp);
      uint2* s_def = s_def_all + kMaxStages * warp;   // entries {slot << 24 | call << 12 | block, dependency + 1}: at most S / P
      const int per_lap = S / P;
      const uint64_t pol_x = l2_policy_evict_last();
      int slot = warp, lap = 0;        // next slot of this pair and how often it has been used
      int t0mod = 0;                   // tiles of all earlier units, modulo P
      int def_head = 0, ndef = 0;      // deferred activation copies: oldest entry (ring index into s_def) and how many
      int dep_ok = -1;                 // the dependency last seen complete
      bool ok = true;
#ifdef BAS_TRACE_PRODUCER
      int trace_flushes = 0, trace_last_call = -1;
#endif

      // Issue the activation copy of the oldest deferred tile; `block`: wait for its call's dependency.
      // `force`: issue it whatever the dependency says (giving up: nobody consumes the tile, but its barrier
      // must complete before the CTA may leave).
      auto flush_one = [&](bool block, bool force) -> bool {   // lane 0 only; false = not ready (or gave up: ok cleared)
        const uint2 e2 = s_def[def_head % kMaxStages];
        const uint32_t e = e2.x;
        const int dslot = (int)(e >> 24), dcall = (int)((e >> 12) & 0xfffu), dj = (int)(e & 0xfffu);
        const ListCallDev* cd = p.calls + dcall;
        const int dep = (int)e2.y - 1;
        if (!force && dep >= 0 && dep != dep_ok) {
          // Copy warp 0 polls the counter in global memory and tells the other copy warps through a
          // word in shared memory (one reader per CTA on the counter's cache line, not four).
          const unsigned int target = (epoch + 1u) * __ldg(&cd->dep_contrib);
          const bool stalled = dcall == p.stall_call;
          unsigned int polls = 0u;
          auto is_ready = [&]() -> bool {
            if (stalled) return false;
            if (warp != 0) {
              if (ld_acquire_cta_shared_u32(&hdr->dep_seen) == (unsigned int)dep + 1u) return true;
              if ((++polls & 7u) != 1u) return false;   // warp 0 may be waiting for another call: look for oneself now and then
            }
            if ((int)(ld_acquire_gpu_u32(p.done + dep) - target) < 0) return false;
            if (warp == 0) st_release_cta_shared_u32(&hdr->dep_seen, (unsigned int)dep + 1u);
            return true;
          };
          bool ready = is_ready();
          if (!ready && block) {
            const long long t_start = clock64();
            while (true) {
              ready = is_ready();
              if (ready) break;
              if (*abort_flag != 0 || clock64() - t_start > limit) {
                ok = false;
                return false;
              }
              __nanosleep(40);
            }
          }
          if (!ready) return false;
          fence_proxy_async_all();   // the tensor copy below reads what other CTAs stored with plain stores
          dep_ok = dep;
          if (warp == 0) BAS_LTRACE(dcall, 1);
        }
#ifdef BAS_TRACE_PRODUCER
        if (warp == 0) BAS_LTRACE_TILE(dcall, trace_flushes, 0);
#endif
        tma_load_2d_hint(s_stage + (size_t)dslot * tile_bytes + p.wslot, &cd->xmap, dj * kBlockK, 0, &hdr->full[dslot], pol_x);
#ifdef BAS_TRACE_PRODUCER
        if (warp == 0) BAS_LTRACE_TILE(dcall, trace_flushes, 1);
        trace_flushes = (dcall == trace_last_call) ? trace_flushes + 1 : 1;
        trace_last_call = dcall;
#endif
        ++def_head;
        --ndef;
        return true;
      };

      // Wait (bounded) until call d has been reported complete by `contrib` CTAs; the whole warp calls this.
      // Activation copies of earlier calls keep going out meanwhile: call d may be waiting for them.
      auto wait_call = [&](int d, unsigned int contrib) -> bool {
        bool ready = true;
        if (lane == 0 && d != dep_ok) {
          const unsigned int target = (epoch + 1u) * contrib;
          const long long t_start = clock64();
          unsigned int polls = 0u;
          for (;;) {
            bool seen = false;
            if (warp != 0 && ld_acquire_cta_shared_u32(&hdr->dep_seen) == (unsigned int)d + 1u) {
              seen = true;
            } else if (warp == 0 || (++polls & 7u) == 1u) {
              if ((int)(ld_acquire_gpu_u32(p.done + d) - target) >= 0) {
                seen = true;
                if (warp == 0) st_release_cta_shared_u32(&hdr->dep_seen, (unsigned int)d + 1u);
              }
            }
            if (seen) break;
            while (ndef > 0 && ok && flush_one(false, false)) {
            }
            if (!ok || *abort_flag != 0 || clock64() - t_start > limit) {
              ready = false;
              break;
            }
            __nanosleep(40);
          }
          if (ready) {
            fence_proxy_async_all();
            dep_ok = d;
          }
        }
        ready = __shfl_sync(0xffffffffu, ready ? 1 : 0, 0) != 0;
        __syncwarp();
        return ready;
      };

      CallRegs cur = load_call_regs(p.calls);
      CallRegs nxt = load_call_regs(p.calls + (p.n_calls > 1 ? 1 : 0));
      int raw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      bool have_raw = false;
      // id batch of a call whose descriptor is in registers (lists with a device-side count are read at the boundary)
      auto prefetch_ids = [&](const CallRegs& r, int (&dst)[8]) -> bool {
        if (regs_ptr(r.b.x, r.b.y) != nullptr) return false;
        if (SEL && ((int)r.c.x < 0 || (int)r.c.z == 0)) return false;   // a mask from an entry, or an entry: no list at all
        const uint8_t* bm = (const uint8_t*)regs_ptr(r.b.z, r.b.w);
        warp_load_id_batch((const int32_t*)regs_ptr(r.a.z, r.a.w), bm, bm != nullptr ? (int)r.c.w : (int)r.c.x, 0, lane, dst);
        return true;
      };
      have_raw = prefetch_ids(cur, raw);

      int c_at = 0;   // the call this role is in (for the status detail of a wait that runs out)
      for (int c = 0; c < p.n_calls && ok; ++c) {
        c_at = c;
        const ListCallDev* cd = p.calls + c;
        const CallRegs nn = load_call_regs(p.calls + (c + 2 < p.n_calls ? c + 2 : c));   // in flight during this call
        const int units = (int)cur.d.x, ranges = (int)cur.d.y, range_off = (int)cur.d.z, dep = (int)cur.d.w;
        const Share sh = call_share(units, ranges, range_off, cid, p.n_clusters);
        int k_mine = 0;
        const bool is_sel = SEL && (int)cur.c.z == 0;                            // a selection entry: no output columns
        const int mask_call = (SEL && (int)cur.c.x < 0) ? -(int)cur.c.x - 1 : -1;   // the entry this call's mask comes from
        if (is_sel) {
          if (sh.part) {
            // This CTA's blocks of the entry (range, range + ranges, ...), dealt out over its copy warps: wait for
            // X, score, publish; the CTA reports once all its copy warps have.
            if (dep >= 0 && !wait_call(dep, cur.b.w)) ok = false;
            if (warp == 0 && lane == 0) BAS_LTRACE(c, 3);
            if (ok) {
              int range = cid - (range_off & kRangeOffMask);
              if (range < 0) range += p.n_clusters;
              // (an entry keeps X, its row stride, the score array and the score kind where a contraction keeps its
              // weights, id list, count and byte map: in the registers fetched two calls ahead)
              const __half* xs = (const __half*)regs_ptr(cur.a.x, cur.a.y);
              double* scores = (double*)regs_ptr(cur.a.z, cur.a.w);
              const long long ldx = (long long)cur.b.x;
              const bool norm = (int)cur.b.z == BAS_SCORE_NORM;
              const int nb_e = (int)cur.c.w, keep_e = (int)cur.c.x;
              const unsigned int own_reports = cur.b.y;
              // a K-sharded activation: this rank's blocks are blocks g0 .. of nb_all, and their scores go to
              // every rank (two self-validating words per block; the stamp is the entry's number in the group)
              const bool sharded = TP && (range_off & kCallSharded) != 0;
              int g0 = 0, nb_all = nb_e;
              unsigned int stamp = 0u;
              if (sharded) {
                g0 = __ldg(&cd->w_rows);
                nb_all = __ldg(&cd->out_compact);
                stamp = sel_base + (unsigned int)__ldg(&cd->tp_index) + 1u;
                if (g0 < 0 || nb_all > kTpSelBlocks || nb_all > p.sel_rep_stride || g0 + nb_e > nb_all) {
                  if (lane == 0) atomicOr(&p.hdr->status, kStatusBadLayout);   // (the host checks these: belt and braces)
                  ok = false;
                }
              }
              bool scored = false;
              for (int j = range + ranges * warp; j < nb_e && ok; j += ranges * P) {
                const double sc = warp_block_score(xs, ldx, (int)cur.c.y, j, bf16, norm, lane);
                if (sharded) {
                  if constexpr (TP) {
                    if (lane < p.tp.world) {
                      const unsigned long long bits = (unsigned long long)__double_as_longlong(sc);
                      unsigned long long* dst = (unsigned long long*)p.tp.area[lane] + p.tp.sel_words + 2 * (size_t)(g0 + j);
                      st_relaxed_sys_u64(dst, ((unsigned long long)stamp << 32) | (bits >> 32));
                      st_relaxed_sys_u64(dst + 1, ((unsigned long long)stamp << 32) | (bits & 0xffffffffull));
                    }
                  }
                } else if (lane < kSelReplicas) {
                  scores[(size_t)lane * (size_t)p.sel_rep_stride + j] = sc;
                }
                scored = true;
              }
              // every copy warp that had a block reports for itself (the copy warps of a CTA do not move in step,
              // so there is no "last of the CTA"); the host knows how many such warps an entry has
              if (warp == 0 && lane == 0) BAS_LTRACE(c, 4);
              if (lane == 0 && scored) red_release_gpu_add_u32(p.done + c, 1u);
              if (warp == 0 && lane == 0) BAS_LTRACE(c, 5);
              // ... and, once every score is there, says for each of its blocks whether it is kept: its rank among
              // all blocks is a handful of comparisons per lane.  The answer goes out as a word that validates
              // itself (the run's number beside the verdict), which the calls that use the mask poll for.
              if (scored && ok) {
                if (!sharded && !wait_call(c, own_reports)) ok = false;
                if (ok) {
                  const double* sc_rep = scores + (size_t)((blockIdx.x * kLProducers + warp) % kSelReplicas) * (size_t)p.sel_rep_stride;
                  unsigned int* flags = (unsigned int*)(scores + (size_t)kSelReplicas * (size_t)p.sel_rep_stride);
                  const unsigned long long* words = nullptr;     // sharded: all ranks' scores, in this rank's own area
                  if constexpr (TP) words = (const unsigned long long*)p.tp.own + p.tp.sel_words;
                  const long long t_start = clock64();
                  // scores of blocks i0 + lane + 32 t; sharded: polled (bounded) until they carry the entry's stamp
                  auto load_scores = [&](int i0, double (&v8)[8]) -> bool {
                    if constexpr (TP) {
                      while (sharded) {      // leaves by a return
                        unsigned long long hi8[8], lo8[8];
                        bool valid = true;
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                          const int i = i0 + lane + 32 * t;
                          hi8[t] = lo8[t] = (unsigned long long)stamp << 32;
                          if (i < nb_all) {
                            hi8[t] = ld_relaxed_sys_u64(words + 2 * (size_t)i);
                            lo8[t] = ld_relaxed_sys_u64(words + 2 * (size_t)i + 1);
                          }
                          valid = valid && (unsigned int)(hi8[t] >> 32) == stamp && (unsigned int)(lo8[t] >> 32) == stamp;
                        }
                        if (__all_sync(0xffffffffu, valid)) {
#pragma unroll
                          for (int t = 0; t < 8; ++t)
                            v8[t] = __longlong_as_double((long long)((hi8[t] << 32) | (lo8[t] & 0xffffffffull)));
                          return true;
                        }
                        bool give_up = false;
                        if (lane == 0) {
                          while (ndef > 0 && ok && flush_one(false, false)) {
                          }
                          give_up = !ok || *abort_flag != 0 || clock64() - t_start > limit;
                        }
                        if (__shfl_sync(0xffffffffu, give_up ? 1 : 0, 0) != 0) return false;
                        __nanosleep(40);
                      }
                    }
#pragma unroll
                    for (int t = 0; t < 8; ++t) v8[t] = (i0 + lane + 32 * t < nb_all) ? __ldcg(sc_rep + i0 + lane + 32 * t) : 0.0;
                    return true;
                  };
                  for (int j = range + ranges * warp; j < nb_e && ok; j += ranges * P) {
                    const int jg = g0 + j;                       // the block's number in the whole input
                    // the block's own key, from the same array as the others (every rank compares the same bits)
                    unsigned long long kj = 0ull;
                    if (!sharded) {
                      kj = score_key(__ldcg(sc_rep + j));
                    } else {
                      double v8[8];
                      const int i0 = jg & ~255;
                      if (!load_scores(i0, v8)) ok = false;
                      double own = 0.0;
#pragma unroll
                      for (int t = 0; t < 8; ++t)
                        if (t == ((jg - i0) >> 5)) own = v8[t];
                      kj = score_key(__shfl_sync(0xffffffffu, own, jg & 31));
                    }
                    int above = 0;
                    for (int i0 = 0; i0 < nb_all && ok; i0 += 256) {     // 256 scores in flight together
                      double v8[8];
                      if (!load_scores(i0, v8)) {
                        ok = false;
                        break;
                      }
#pragma unroll
                      for (int t = 0; t < 8; ++t) {
                        const int i = i0 + lane + 32 * t;
                        const unsigned long long ki = score_key(v8[t]);
                        above += (i < nb_all && (ki > kj || (ki == kj && i < jg))) ? 1 : 0;
                      }
                    }
                    if (!ok) break;
                    above = __reduce_add_sync(0xffffffffu, above);
                    const unsigned int word = (((epoch + 1u) & 0x7fffffffu) << 1) | (above < keep_e ? 1u : 0u);
                    if (lane < kSelReplicas) st_release_gpu_u32(flags + (size_t)lane * (size_t)p.sel_rep_stride + jg, word);
                  }
                }
              }
            }
          }
        } else if (sh.part) {
          int k_act = 0;
          if (mask_call >= 0) {
            // (such a call keeps the entry's score array, from which the verdicts follow, {blocks of the entry},
            // and its first block of the mask where the others keep id list, count and byte map)
            // One word per block of the entry, written by whoever scored the block: valid once it carries this
            // run's number.  Poll (bounded) until all are; earlier calls' activation copies keep going out meanwhile.
            const int mnb = (int)(cur.b.x & 0xffffu), mblock0 = (int)cur.b.z;
            const unsigned int* flags = (const unsigned int*)((const double*)regs_ptr(cur.a.z, cur.a.w) + (size_t)kSelReplicas * (size_t)p.sel_rep_stride) +
                                        (size_t)((blockIdx.x * kLProducers + warp) % kSelReplicas) * (size_t)p.sel_rep_stride;
            const unsigned int want = (epoch + 1u) & 0x7fffffffu;
            int32_t* ids_out = (warp == 0 && rank == 0 && sh.n0 == 0) ? ldg_ptr(&cd->ids_out) : nullptr;
            const long long t_start = clock64();
            int total = 0;
            // (an entry over a sharded activation: this rank has the verdicts of its own blocks only)
            const bool own_only = (range_off & kCallSharded) != 0;
            const int f_lo = own_only ? mblock0 : 0, f_hi = own_only ? mblock0 + (int)cur.c.w : mnb;
            if (f_lo < 0 || f_hi > p.sel_rep_stride || f_hi <= f_lo) {
              if (lane == 0) atomicOr(&p.hdr->status, kStatusBadLayout);
              ok = false;
            }
            for (int i0 = f_lo; i0 < f_hi && ok; i0 += 256) {
              unsigned int w8[8];
              for (;;) {
                bool valid = true;
#pragma unroll
                for (int t = 0; t < 8; ++t) {      // relaxed loads: all of a lane's words are in flight together
                  const int i = i0 + lane + 32 * t;
                  w8[t] = (i < f_hi) ? ld_relaxed_gpu_u32(flags + i) : (want << 1);
                  valid = valid && (w8[t] >> 1) == want;
                }
                if (__all_sync(0xffffffffu, valid)) {
                  // One acquire, of any valid word: its writer had seen X complete (it acquired the counter of the
                  // call that writes X before it scored), which is all this call needs beyond the words themselves.
                  if (i0 == f_lo) (void)ld_acquire_gpu_u32(flags + f_lo + lane % (f_hi - f_lo));
                  break;
                }
                bool give_up = false;
                if (lane == 0) {
                  while (ndef > 0 && ok && flush_one(false, false)) {
                  }
                  give_up = !ok || *abort_flag != 0 || clock64() - t_start > limit;
                }
                if (__shfl_sync(0xffffffffu, give_up ? 1 : 0, 0) != 0) {
                  ok = false;
                  break;
                }
                __nanosleep(40);
              }
              if (!ok) break;
#pragma unroll
              for (int t = 0; t < 8; ++t) {
                const int i = i0 + lane + 32 * t;
                if (i0 + 32 * t < f_hi) {      // (uniform)
                  const bool sel = i < f_hi && (w8[t] & 1u) != 0u;
                  const bool loc = sel && i >= mblock0 && i < mblock0 + (int)cur.c.w;
                  const unsigned int ms = __ballot_sync(0xffffffffu, sel), ml = __ballot_sync(0xffffffffu, loc);
                  const unsigned int below = (1u << lane) - 1u;
                  if (loc) s_ids[k_act + __popc(ml & below)] = (uint16_t)(i - mblock0);
                  if (sel && ids_out != nullptr) ids_out[total + __popc(ms & below)] = i;
                  total += __popc(ms);
                  k_act += __popc(ml);
                }
              }
            }
            __syncwarp();
            if (warp == 0 && lane == 0) BAS_LTRACE(mask_call, 7);
            if (ok && lane == 0) {
              fence_proxy_async_all();
              dep_ok = dep;     // whoever wrote the verdicts had seen X complete: so has this warp now
            }
          } else {
            k_act = warp_stage_ids((const int32_t*)regs_ptr(cur.a.z, cur.a.w), (const int32_t*)regs_ptr(cur.b.x, cur.b.y),
                                   (int)cur.c.x, (const uint8_t*)regs_ptr(cur.b.z, cur.b.w), (int)cur.c.w, s_ids,
                                   &p.hdr->status, lane, have_raw, raw, warp == 0 && rank == 0 && sh.n0 == 0);
          }
          k_mine = (k_act > rank) ? (k_act - rank + C - 1) / C : 0;
        }
        if (warp == 0 && lane == 0) {
          // An MMA costs the tensor core by the rows of the weight operand it reads (measured: 39
          // cycles per M = 128 instruction, 23 per M = 64): tiles of up to 64 columns use the short form.
          // (A selection entry is the copy warps' business alone: the other warps skip it.)
          s_rec[c] = make_record(sh.part && !is_sel, C == 1 && sh.tw <= 64, sh.n_sub, k_mine);
          st_release_cta_shared_u32(&hdr->calls_staged, (unsigned int)(c + 1));
        }
        // the next call's id list: requested now, used at the next boundary
        int raw_n[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const bool have_n = (c + 1 < p.n_calls) ? prefetch_ids(nxt, raw_n) : false;
        if (warp == 0 && lane == 0) BAS_LTRACE(c, 0);
        if (lane == 0 && sh.part && !is_sel && k_mine > 0) {
          const uint8_t* packed = (const uint8_t*)regs_ptr(cur.a.x, cur.a.y);
          int npad = units * 8;
          const bool by_block = SEL && (range_off & kCall2d) != 0;          // output-block sparsity
          const bool x_compact = SEL && (range_off & kCallXCompact) != 0;   // X holds the active blocks only
          const int32_t* n_ids = nullptr;
          if (by_block) {
            npad = __ldg(&cd->w_rows);
            n_ids = ldg_ptr(&cd->n_ids);
          }
          for (int sub = 0; sub < sh.n_sub && ok; ++sub) {
            int c0 = sh.n0 + sub * sh.tw;
            int wbytes = min(sh.tw, sh.width - sub * sh.tw) * kRowBytes;
            if (by_block) {
              // this tile's weights are the rows of output block n_ids[q] (a bad id is reported by the epilogue
              // and read as the nearest valid block: nothing outside the weight is touched)
              const int o = min(max(__ldg(n_ids + (c0 >> 6)), 0), (npad - 1) >> 6);
              c0 = o * 64;
              wbytes = min(64, npad - c0) * kRowBytes;
            }
            int i = warp - t0mod;
            if (i < 0) i += P;
            for (; i < k_mine; i += P) {
              // the slot about to be reused may still hold a tile whose activations were never
              // requested: that one has to go out first, whatever it waits for
              if (ndef >= per_lap) {
                while (ndef >= per_lap && ok) (void)flush_one(true, false);
                while (ndef > 0 && ok && flush_one(false, false)) {   // and with it everything else that has become ready
                }
              }
              if (!ok) break;
              if (lap > 0 && !mbar_wait_for(&hdr->empty[slot], (lap - 1) & 1, abort_flag, limit)) {
                ok = false;
                break;
              }
              const int j = s_ids[rank + i * C];
              mbar_arrive_expect_tx(&hdr->full[slot], wbytes + kXTileBytes);
              uint8_t* st = s_stage + (size_t)slot * tile_bytes;
              bulk_copy_g2s(st, packed + ((size_t)j * npad + c0) * kRowBytes, wbytes, &hdr->full[slot]);
              ++armed_cnt;
              const int xb = x_compact ? rank + i * C : j;     // the block of X that goes with this tile
              if (ndef == 0 && (dep < 0 || dep == dep_ok)) {
                tma_load_2d_hint(st + p.wslot, &cd->xmap, xb * kBlockK, 0, &hdr->full[slot], pol_x);
              } else {
                s_def[(def_head + ndef) % kMaxStages] =
                    make_uint2(((uint32_t)slot << 24) | ((uint32_t)c << 12) | (uint32_t)xb, (uint32_t)(dep + 1));
                ++ndef;
                while (ndef > 0 && flush_one(false, false)) {
                }
              }
              slot += P;
              if (slot >= S) {
                slot -= S;
                ++lap;
              }
            }
            t0mod += k_mine % P;
            if (t0mod >= P) t0mod -= P;
          }
        }
        if (warp == 0 && lane == 0) BAS_LTRACE(c, 2);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        cur = nxt;
        nxt = nn;
        have_raw = have_n;
#pragma unroll
        for (int e = 0; e < 8; ++e) raw[e] = raw_n[e];
      }
      if (lane == 0) {
        while (ndef > 0 && ok) (void)flush_one(true, false);
        if (!ok) {
          if (atomicExch(&hdr->abort_flag, 1) == 0) record_expiry(&p.hdr->status, kWhereCopyWarp, c_at);   // the first of this CTA: the others only follow it
          while (ndef > 0) (void)flush_one(false, true);
        }
      }
      __syncwarp();
    }
    if (warp == 0) pdl_launch_dependents();
  } else if (warp < kLEpiWarp0) {
    // ================================ MMA issuers ================================
    const int w = warp - kLProducers;
    if (lane == 0 && w < PI) {
      bool ok = true;
      int slot = w % S, fph = (w / S) & 1, t0mod = 0, u = 0;
      int c_at = 0;   // the call this role is in (for the status detail of a wait that runs out)
      for (int c = 0; c < p.n_calls && ok; ++c) {
        c_at = c;
        // the call's record: published by copy warp 0 before it issues the call's first tile
        if (ld_acquire_cta_shared_u32(&hdr->calls_staged) <= (unsigned int)c) {
          const long long t_start = clock64();
          while (ld_acquire_cta_shared_u32(&hdr->calls_staged) <= (unsigned int)c) {
            if (*abort_flag != 0 || clock64() - t_start > limit) {
              ok = false;
              break;
            }
          }
          if (!ok) break;
        }
        const unsigned int rec = s_rec[c];
        if ((rec & 0x80000000u) == 0u) continue;
        const int n_sub = (int)((rec >> 16) & 0xffu), k_mine = (int)(rec & 0xffffu);
        const uint32_t idesc = (rec & 0x40000000u) != 0u ? kIdesc64 : kIdesc;
        for (int sub = 0; sub < n_sub && ok; ++sub, ++u) {
          const int b = u & 1;
          // the accumulator buffer is free once the epilogue has read out unit u - 2; passing this
          // wait also means that every issuer has signed off that unit
          if (u >= 2 && !mbar_wait_for(&hdr->acc_empty[b], ((u >> 1) - 1) & 1, abort_flag, limit)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t d = tmem_base + (uint32_t)((b * kAccIssuers + w) * BPAD);
          bool fresh = true;
          int i = w - t0mod;
          if (i < 0) i += PI;
          for (; i < k_mine; i += PI) {
            if (!mbar_wait_for(&hdr->full[slot], fph, abort_flag, limit)) {
              ok = false;
              break;
            }
            // (no tcgen05 fence here: the tile was written by bulk copies and observed through the barrier; the
            // fence after the accumulator hand-over above is the only ordering against other threads' tcgen05
            // operations that the MMAs need, and one fence per tile cost the issuer about 0.3 us each)
            if (w == 0 && fresh && sub == 0) BAS_LTRACE(c, 3);
#ifdef BAS_TRACE
            if (w == 0 && p.trace != nullptr && blockIdx.x == p.trace_cta && c < BAS_LTRACE_CALLS && i / PI < 4) {
              // low bits of the stamp: which of this issuer's next three slots already hold their tile
              unsigned long long gt_;
              asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));
              unsigned long long mask = 0;
              int s2 = slot, ph2 = fph;
              for (int q = 0; q < 3; ++q) {
                s2 += PI;
                if (s2 >= S) { s2 -= S; ph2 ^= 1; }
                if (mbar_test_wait(&hdr->full[s2], ph2)) mask |= 1ull << q;
              }
              p.trace[(BAS_LTRACE_CALLS + c) * BAS_LTRACE_EVENTS + 2 * (i / PI)] = (long long)((gt_ & ~7ull) | mask);
            }
#endif
            const uint32_t st = smem_u32(s_stage + (size_t)slot * tile_bytes);
            const uint64_t adesc = umma_desc_kmajor_sw128(st);
            const uint64_t bdesc = umma_desc_kmajor_sw128(st + p.wslot);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_f16_ss(d, adesc + (uint64_t)(2 * ks), bdesc + (uint64_t)(2 * ks), idesc, (fresh && ks == 0) ? 0u : 1u);
            fresh = false;
            umma_commit(&hdr->empty[slot]);   // the slot is free once these MMAs have read it
#ifndef BAS_TRACE_PRODUCER
            if (w == 0) BAS_LTRACE_TILE(c, i / PI, 1);
#endif
            slot += PI;
            if (slot >= S) {
              slot -= S;
              fph ^= 1;
            }
          }
          if (!ok) break;
          if (!fresh) umma_commit(&hdr->acc_full[b]);
          else mbar_arrive(&hdr->acc_full[b]);
          if (w == 0 && sub == n_sub - 1) BAS_LTRACE(c, 4);
          t0mod += k_mine % PI;
          if (t0mod >= PI) t0mod -= PI;
        }
      }
      if (!ok) {
        if (atomicExch(&hdr->abort_flag, 1) == 0) record_expiry(&p.hdr->status, kWhereIssuer, c_at);   // the first of this CTA: the others only follow it
      }
    }
  } else {
    // ================================ epilogue ================================
    const int q = warp & 3;
    const int et = tid - 32 * kLEpiWarp0;
    constexpr int kChunks = BPAD / 16;
    constexpr int kChunks0 = (kChunks + 1) / 2;
    bool ok = true;
    unsigned int where = kWhereEpilogue;     // which of the epilogue's waits ran out first (status bits 8..)
    int t0mod = 0, u = 0;
    int n_part = 0;                          // calls this CTA has taken part in so far
    int c_at = 0;   // the call this role is in (for the status detail of a wait that runs out)
    for (int c = 0; c < p.n_calls && ok; ++c) {
      c_at = c;
      {
        bool ready = ld_acquire_cta_shared_u32(&hdr->calls_staged) > (unsigned int)c;
        if (!__all_sync(0xffffffffu, ready)) {
          const long long t_start = clock64();
          while (true) {
            ready = ld_acquire_cta_shared_u32(&hdr->calls_staged) > (unsigned int)c;
            const bool give_up = *abort_flag != 0 || clock64() - t_start > limit;
            if (__all_sync(0xffffffffu, ready)) break;
            if (__any_sync(0xffffffffu, give_up)) {
              ok = false;
              break;
            }
          }
          if (!ok) break;
        }
      }
      const unsigned int rec = s_rec[c];
      if ((rec & 0x80000000u) == 0u) continue;
      const int k_mine = (int)(rec & 0xffffu);
      // Row of the accumulator (= column within the tile) that this thread reads: M = 128 fills all
      // 128 lanes of tensor memory; M = 64 puts rows 16q .. 16q+15 on the first 16 lanes of quarter q.
      const int r = (rec & 0x40000000u) != 0u ? (lane < 16 ? 16 * q + lane : kTileN) : q * 32 + lane;
      const ListCallDev* cd = p.calls + c;
      const Share sh = call_share(__ldg(&cd->units), __ldg(&cd->ranges), __ldg(&cd->range_off), cid, p.n_clusters);
      __half* y = ldg_ptr(&cd->y);
      const long long ldy = __ldg(&cd->ldy);
      const int batch = __ldg(&cd->batch), n = __ldg(&cd->n);
      // Row-parallel call: the tile's fp32 partials of every rank go to ONE rank (the tile's owner, by
      // tile index), which adds them in rank order, rounds once and sends the 16-bit results to the
      // others (reduce-scatter, then gather): two NVLink traversals, 1 / world of the bytes of sending
      // every partial to every rank.  All words are 64-bit {payload, exchange number}: a reader polls
      // its own memory until the number is the current one; no flags, no fences.
      int tp_k = -1, tp_owner = 0;
      unsigned int tp_epoch = 0u;
      size_t tp_buf = 0;          // word offset of the current receive buffer inside any rank's area
      if constexpr (TP) {
        tp_k = __ldg(&cd->tp_index);
        if (tp_k >= 0) {
          tp_epoch = tp_base + (unsigned int)tp_k + 1u;
          tp_buf = (size_t)kTpHeaderBytes / 8 + (size_t)(tp_epoch & 1u) * (size_t)p.tp.world * (size_t)p.tp.src_words;
          int range = cid - (__ldg(&cd->range_off) & kRangeOffMask);
          if (range < 0) range += p.n_clusters;
          tp_owner = range % p.tp.world;
          // No active block on this rank: no activation copy made this CTA wait for the call's dependency, yet
          // its zeros must not leave before it.  The exchange before last used the same words, and only the
          // chain of dependencies from one row-parallel call to the next says that every rank has read them.
          const int dep = __ldg(&cd->dep);
          if (k_mine == 0 && dep >= 0) {
            const unsigned int target = (epoch + 1u) * __ldg(&cd->dep_contrib);
            bool ready = true;
            if (lane == 0) {
              const long long t_start = clock64();
              while (c == p.stall_call || (int)(ld_acquire_gpu_u32(p.done + dep) - target) < 0) {
                if (*abort_flag != 0 || clock64() - t_start > limit) {
                  ready = false;
                  break;
                }
                __nanosleep(100);
              }
            }
            if (!__all_sync(0xffffffffu, ready)) {
              ok = false;
              break;
            }
          }
        }
      }

      const bool by_block = SEL && (__ldg(&cd->range_off) & kCall2d) != 0;    // output-block sparsity
      const int32_t* n_ids = by_block ? ldg_ptr(&cd->n_ids) : nullptr;
      const bool out_compact = by_block && __ldg(&cd->out_compact) != 0;
      for (int sub = 0; sub < sh.n_sub && ok; ++sub, ++u) {
        const int b = u & 1;
        const int c0 = sh.n0 + sub * sh.tw;
        const int wsub = min(sh.tw, sh.width - sub * sh.tw);
        // where the tile's columns are in the weight (for the bound against n) and where they go in y
        int wcol0 = c0, ycol0 = c0;
        if (by_block) {
          const int o_raw = __ldg(n_ids + (c0 >> 6)), o_max = (n - 1) >> 6;
          if ((o_raw < 0 || o_raw > o_max) && et == 0) atomicOr(&p.hdr->status, BAS_DEV_BAD_BLOCK_ID);
          wcol0 = min(max(o_raw, 0), o_max) * 64;
          if (!out_compact) ycol0 = wcol0;
        }
        if (!__all_sync(0xffffffffu, mbar_wait_for(&hdr->acc_full[b], (u >> 1) & 1, abort_flag, limit))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (et == 0 && sub == sh.n_sub - 1) BAS_LTRACE(c, 5);
        float* red_buf = s_red + (size_t)b * BPAD * kTileN;

        auto emit = [&](auto ch0_c, auto nch_c) {
          constexpr int CH0 = decltype(ch0_c)::value, NCH = decltype(nch_c)::value;
          constexpr int NV = NCH * 16;
          constexpr int IB = (BPAD == 16) ? 4 : (NCH == 1) ? 2 : 1;
          float v[NV];
#pragma unroll
          for (int e = 0; e < NV; ++e) v[e] = 0.f;
          if (k_mine > 0) {
#pragma unroll
            for (int w0 = 0; w0 < kAccIssuers; w0 += IB) {
              if (w0 < PI) {
                uint32_t regs[IB][NCH][16];
#pragma unroll
                for (int wi = 0; wi < IB; ++wi)
                  if (w0 + wi < PI) {
#pragma unroll
                    for (int cc = 0; cc < NCH; ++cc)
                      tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) +
                                             (uint32_t)((b * kAccIssuers + w0 + wi) * BPAD + (CH0 + cc) * 16),
                                         regs[wi][cc]);
                  }
                tmem_ld_wait();
#pragma unroll
                for (int wi = 0; wi < IB; ++wi) {
                  const int w = w0 + wi;
                  int first = w - t0mod;      // this issuer's first tile of the unit
                  if (first < 0) first += PI;
                  if (w < PI && first < k_mine) {   // issuer order: the sum never depends on timing
#pragma unroll
                    for (int cc = 0; cc < NCH; ++cc)
#pragma unroll
                      for (int e = 0; e < 16; ++e) v[cc * 16 + e] += __uint_as_float(regs[wi][cc][e]);
                  }
                }
              }
            }
          }
          if (TP && tp_k >= 0) {
            // this rank's partial of column c0 + r, to the tile's owner (padded columns too: they are zero)
            if (r < wsub) {
              unsigned long long* dst = (unsigned long long*)p.tp.area[tp_owner] + tp_buf +
                                        (size_t)p.tp.rank * (size_t)p.tp.src_words + (size_t)(c0 + r);
#pragma unroll
              for (int e = 0; e < NV; ++e)
                if (16 * CH0 + e < batch)
                  st_relaxed_sys_u64(dst + (size_t)(16 * CH0 + e) * (size_t)p.tp.ldp,
                                     ((unsigned long long)tp_epoch << 32) | (unsigned long long)__float_as_uint(v[e]));
            }
          } else if (C == 1) {
            const int col = ycol0 + r;
            if (r < wsub && wcol0 + r < n) {
#pragma unroll
              for (int e = 0; e < NV; ++e)
                if (16 * CH0 + e < batch) store_out16(y + (size_t)(16 * CH0 + e) * ldy + col, v[e], bf16);
            }
          } else {
            // batch row b is finished by rank b % C: push this CTA's partial of each row into the
            // owner's receive buffer [source rank][column][row slot], four row slots per 16-byte store
            const int nbi = BPAD / C;
            const int sw = red_swizzle_l(nbi, r);
            float* mine_l = red_buf + (rank * kTileN + r) * nbi;
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
                  if (16 * b4 + o < batch) {
                    const float4 val = make_float4(v[16 * c4 + o], v[16 * c4 + o + 4], v[16 * c4 + o + 8], v[16 * c4 + o + 12]);
                    if (o == rank) *(float4*)(mine_l + 4 * (b4 ^ sw)) = val;
                    else dsmem_st_v4_f32(owner[o] + (uint32_t)(16 * (b4 ^ sw)), val.x, val.y, val.z, val.w);
                  }
                }
            } else {
#pragma unroll
              for (int o = 0; o < 2; ++o)
#pragma unroll
                for (int c8 = 0; c8 < 2 * NCH; ++c8) {   // slots 4*b8 .. 4*b8+3 <-> rows 8*b8 + o + {0,2,4,6}
                  const int b8 = 2 * CH0 + c8;
                  if (8 * b8 + o < batch) {
                    const float4 val = make_float4(v[8 * c8 + o], v[8 * c8 + o + 2], v[8 * c8 + o + 4], v[8 * c8 + o + 6]);
                    if (o == rank) *(float4*)(mine_l + 4 * (b8 ^ sw)) = val;
                    else dsmem_st_v4_f32(owner[o] + (uint32_t)(16 * (b8 ^ sw)), val.x, val.y, val.z, val.w);
                  }
                }
            }
          }
        };
        using std::integral_constant;
        // the batch rows in two rounds of at most 32 (the registers of one round hold 16 values per row chunk)
        if constexpr (kChunks == 1) {
          emit(integral_constant<int, 0>{}, integral_constant<int, 1>{});
        } else {
          emit(integral_constant<int, 0>{}, integral_constant<int, kChunks0>{});
          emit(integral_constant<int, kChunks0>{}, integral_constant<int, kChunks - kChunks0>{});
        }
        // the accumulators have been read: the issuers may overwrite this buffer (unit u + 2)
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->acc_empty[b]);

        if (TP && tp_k >= 0) {
          // ---- the exchange: (row, column pair) elements of the tile dealt out over the 128 threads ----
          const int ppr = wsub >> 1, total = batch * ppr;
          const int world = p.tp.world, me = p.tp.rank;
          const unsigned long long* own = (const unsigned long long*)p.tp.own + tp_buf;
          const long long t_start = clock64();
          bool good = true;
          for (int e0 = et; e0 < total && good; e0 += kLEpiThreads) {
            const int row = e0 / ppr, pc = e0 - row * ppr;
            const int col = c0 + 2 * pc;
            unsigned short h0, h1;
            if (tp_owner == me) {
              // owner: wait for every rank's two partials, add them in rank order, round, keep, send on
              const size_t off = (size_t)row * (size_t)p.tp.ldp + (size_t)col;
              unsigned long long wa[kTpMaxRanks], wb[kTpMaxRanks];
#pragma unroll
              for (int q = 0; q < kTpMaxRanks; ++q) {
                wa[q] = (q < world) ? ld_relaxed_sys_u64(own + (size_t)q * (size_t)p.tp.src_words + off) : 0ull;
                wb[q] = (q < world) ? ld_relaxed_sys_u64(own + (size_t)q * (size_t)p.tp.src_words + off + 1) : 0ull;
              }
              float sa = 0.f, sb = 0.f;
#pragma unroll
              for (int q = 0; q < kTpMaxRanks; ++q)
                if (q < world) {
                  while ((unsigned int)(wa[q] >> 32) != tp_epoch || (unsigned int)(wb[q] >> 32) != tp_epoch) {
                    if (*abort_flag != 0 || clock64() - t_start > limit) {
                      good = false;
                      break;
                    }
                    __nanosleep(32);
                    wa[q] = ld_relaxed_sys_u64(own + (size_t)q * (size_t)p.tp.src_words + off);
                    wb[q] = ld_relaxed_sys_u64(own + (size_t)q * (size_t)p.tp.src_words + off + 1);
                  }
                  sa += __uint_as_float((unsigned int)wa[q]);
                  sb += __uint_as_float((unsigned int)wb[q]);
                }
              if (!good) break;
              h0 = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(sa)) : __half_as_ushort(__float2half_rn(sa));
              h1 = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(sb)) : __half_as_ushort(__float2half_rn(sb));
              const unsigned long long word = ((unsigned long long)tp_epoch << 32) | ((unsigned long long)h1 << 16) | (unsigned long long)h0;
              // results travel in the words [row][c0 + pair] of the slot "source = owner" of every other rank
              const size_t roff = (size_t)me * (size_t)p.tp.src_words + (size_t)row * (size_t)p.tp.ldp + (size_t)(c0 + pc);
#pragma unroll 1
              for (int q = 0; q < world; ++q)
                if (q != me) st_relaxed_sys_u64((unsigned long long*)p.tp.area[q] + tp_buf + roff, word);
            } else {
              const unsigned long long* src = own + (size_t)tp_owner * (size_t)p.tp.src_words + (size_t)row * (size_t)p.tp.ldp + (size_t)(c0 + pc);
              unsigned long long word = ld_relaxed_sys_u64(src);
              while ((unsigned int)(word >> 32) != tp_epoch) {
                if (*abort_flag != 0 || clock64() - t_start > limit) {
                  good = false;
                  break;
                }
                __nanosleep(32);
                word = ld_relaxed_sys_u64(src);
              }
              if (!good) break;
              h0 = (unsigned short)(word & 0xffffull);
              h1 = (unsigned short)((word >> 16) & 0xffffull);
            }
            unsigned short* yrow = reinterpret_cast<unsigned short*>(y) + (size_t)row * (size_t)ldy;
            if (col < n) yrow[col] = h0;
            if (col + 1 < n) yrow[col + 1] = h1;
          }
          if (!__all_sync(0xffffffffu, good)) {
            where = (tp_owner == p.tp.rank) ? kWhereExchangeOwner : kWhereExchangeReader;
            ok = false;
            break;
          }
        }
        if (C > 1) {
          // tell every owner that this warp's pushes are on their way (release at cluster scope, after
          // the warp's stores), then wait until all warps of all CTAs of the cluster have told this one
          if (lane == 0) {
            fence_acq_rel_cluster();
            const uint32_t bar = smem_u32(&hdr->red_full[b]);
            for (int o = 0; o < C; ++o) mbar_arrive_remote(dsmem_addr(bar, (uint32_t)o));
          }
          if (!__all_sync(0xffffffffu, mbar_wait_cluster_for(&hdr->red_full[b], (u >> 1) & 1, abort_flag, limit))) {
            ok = false;
            break;
          }
          const int rr = et & 127;
          const int nbi = BPAD / C;
          const int sw = red_swizzle_l(nbi, rr);
          const int col = c0 + rr;
          if (rr < wsub && col < n) {
            for (int qd = 0; 4 * qd * C + rank < batch; ++qd) {
              float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int s = 0; s < 4; ++s)
                if (s < C) {   // rank order
                  const float4 t = *(const float4*)(red_buf + (s * kTileN + rr) * nbi + 4 * (qd ^ sw));
                  sum.x += t.x;
                  sum.y += t.y;
                  sum.z += t.z;
                  sum.w += t.w;
                }
              const int row0 = 4 * qd * C + rank;
              const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (row0 + e * C < batch) store_out16(y + (size_t)(row0 + e * C) * ldy + col, vals[e], bf16);
            }
          }
        }
        t0mod += k_mine % PI;
        if (t0mod >= PI) t0mod -= PI;
      }
      if (!ok) break;
      // This CTA's part of call c is in global memory: report it, once per CTA.  Every warp arrives on a
      // counter in shared memory (release at CTA scope, after its lanes' stores, which precede the
      // arrival through the warp barrier); the last of them adds one to the call's counter in
      // global memory with release semantics at GPU scope, which covers the other warps' stores as well
      // (they happen before it).  Nothing blocks, so a warp that gave up cannot strand the others, and
      // no separate fence is needed: the readers acquire the counter.
      __syncwarp();
      if (et == 0) BAS_LTRACE(c, 6);
      if (lane == 0 && (atom_add_acq_rel_cta_shared_u32(&hdr->epi_arrived[n_part & 3], 1u) % (kLEpiThreads / 32)) == kLEpiThreads / 32 - 1) {
        red_release_gpu_add_u32(p.done + c, 1u);
        BAS_LTRACE(c, 7);
      }
      ++n_part;
    }
    if (!ok) {
      if (atomicExch(&hdr->abort_flag, 1) == 0) record_expiry(&p.hdr->status, where, c_at);   // the first of this CTA: the others only follow it
    }
  }

  // ---- common tail ----
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (hdr->abort_flag != 0 && warp < P && lane == 0) {
    // Gave up somewhere: do not leave while copies may still be landing in this CTA's memory (every
    // armed tile has had both its copies issued by now): wait, bounded, for this warp's last lap of slots.
    int zero = 0;
    const int per_lap = S / P;
    int k = armed_cnt - 1;
    for (int i = 0; i < per_lap && k >= 0; ++i, --k) {
      const int g = warp + k * P;
      (void)mbar_wait_for(&hdr->full[g % S], (g / S) & 1, &zero, 2000000);
    }
  }
  __syncthreads();
  if (C > 1) cluster_sync_all();   // no CTA leaves while a peer may still push into it or arrive on its barriers
  if (warp == kLEpiWarp0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0) {
    // the last CTA of the run advances the epoch: the counters keep growing, the targets with them
    __threadfence();
    if (atomicAdd(&p.hdr->arrived, 1u) == gridDim.x - 1) {
      p.hdr->arrived = 0u;
      p.hdr->epoch = epoch + 1u;
      if constexpr (TP) {
        ((unsigned int*)p.tp.own)[0] = tp_base + (unsigned int)p.n_tp_calls;
        ((unsigned int*)p.tp.own)[2] = sel_base + (unsigned int)p.n_sharded;
      }
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
constexpr size_t kLSmemBudget = 224 * 1024;

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Shared memory in front of the ring, as the kernel carves it up.
size_t list_fixed_smem(int n_calls, int nb_max, int cluster, int bpad) {
  return 128 + round_up(sizeof(ListSmemHeader), 128) + round_up((size_t)n_calls * 4, 128) +
         round_up((size_t)nb_max * 2, 128) * kLProducers + sizeof(uint2) * kMaxStages * kLProducers +

         (cluster > 1 ? 2 * (size_t)bpad * kTileN * sizeof(float) : 0) + 1024;
}

template <int BPAD>
cudaError_t list_prepare_kernel() {
  static bool done[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(umma_list_kernel<BPAD, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_list_kernel<BPAD, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_list_kernel<BPAD, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(umma_list_kernel<BPAD, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64) done[dev] = true;
  return cudaSuccess;
}

template <int BPAD>
int list_resident_clusters(int cluster, size_t smem, int sm_count) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sm_count / cluster * cluster));
  cfg.blockDim = dim3(kLThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster > 1 ? 1 : 0;
  int n = 0;
  if (cluster == 1) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, umma_list_kernel<BPAD, false, false>, kLThreads, smem) != cudaSuccess) {
      (void)cudaGetLastError();
      return 0;
    }
    return per_sm > 0 ? sm_count : 0;
  }
  if (cudaOccupancyMaxActiveClusters(&n, umma_list_kernel<BPAD, false, false>, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  return n;
}

template <int BPAD>
cudaError_t list_launch(const ListParams& p, size_t smem, cudaStream_t stream) {
  if (p.tp.world > 0)
    return p.extended != 0
               ? launch_with_pdl(umma_list_kernel<BPAD, true, true>, p.n_clusters * p.cluster, kLThreads, smem, p.cluster, stream, p)
               : launch_with_pdl(umma_list_kernel<BPAD, true, false>, p.n_clusters * p.cluster, kLThreads, smem, p.cluster, stream, p);
  return p.extended != 0
             ? launch_with_pdl(umma_list_kernel<BPAD, false, true>, p.n_clusters * p.cluster, kLThreads, smem, p.cluster, stream, p)
             : launch_with_pdl(umma_list_kernel<BPAD, false, false>, p.n_clusters * p.cluster, kLThreads, smem, p.cluster, stream, p);
}

}  // namespace
}  // namespace bas

using namespace bas;

struct bas_list {
  int n_calls = 0, bpad = 0, sm_count = 0;
  size_t smem = 0;
  void* dev_block = nullptr;   // header, counters, descriptors, the selection entries' scores and verdicts
  size_t dev_bytes = 0;
  size_t sel_off = 0;          // where the last of these start
  ListParams params = {};
};

namespace {

template <typename F>
auto by_bpad(int bpad, F&& f) {
  switch (bpad) {
    case 16: return f(std::integral_constant<int, 16>{});
    case 32: return f(std::integral_constant<int, 32>{});
    case 48: return f(std::integral_constant<int, 48>{});
    default: return f(std::integral_constant<int, 64>{});
  }
}

inline bool list_aligned16(const void* ptr) { return (((uintptr_t)ptr) & 15u) == 0; }

}  // namespace

extern "C" {

static int list_create_impl(bas_list** out, const bas_list_call* calls, int n_calls, int flags, const bas_tp* tp);

BAS_API int bas_list_create(bas_list** out, const bas_list_call* calls, int n_calls, int flags) {
  return list_create_impl(out, calls, n_calls, flags, nullptr);
}

BAS_API int bas_list_create_tp(bas_list** out, const bas_list_call* calls, int n_calls, int flags, bas_tp* tp) {
  if (tp == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  return list_create_impl(out, calls, n_calls, flags, tp);
}

static int list_create_impl(bas_list** out, const bas_list_call* calls, int n_calls, int flags, const bas_tp* tp) {
  if (out == nullptr || calls == nullptr || n_calls <= 0) return BAS_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  if (n_calls > BAS_LIST_MAX_CALLS) return BAS_ERR_UNSUPPORTED;
  if (flags < 0 || (flags & ~(BAS_GEMM_BF16 | 0x700 | 0x7000 | 0xff0000 | 0x3f000000)) != 0) return BAS_ERR_INVALID_ARGUMENT;
  int dev = 0, sm_count = 0, cc_major = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (cc_major != 10) return BAS_ERR_UNSUPPORTED;

  // ---- argument checks (those of bas_gemm, per call) and the list-wide sizes ----
  int max_batch = 0, nb_max = 1, sel_nb_max = 0, n_sel = 0, n_gemm = 0, n_shaped = 0, n_sharded = 0;
  for (int c = 0; c < n_calls; ++c) {
    const bas_list_call& a = calls[c];
    if (a.op == BAS_LIST_SELECT) {
      // a selection entry: X, its shape, how many blocks to keep, what it waits for - and nothing else
      if (a.x_dev == nullptr || a.batch <= 0 || a.k < kBlockK || (a.k % kBlockK) != 0 || a.ldx < a.k) return BAS_ERR_INVALID_ARGUMENT;
      if (a.batch > BAS_MAX_BATCH || a.k / kBlockK > BAS_LIST_MAX_BLOCKS) return BAS_ERR_UNSUPPORTED;
      const bool sharded = (a.shape_flags & BAS_LIST_SELECT_SHARDED) != 0;
      if ((a.shape_flags & ~BAS_LIST_SELECT_SHARDED) != 0) return BAS_ERR_INVALID_ARGUMENT;
      if (sharded) {
        // X is this rank's K-shard: blocks mask_block0 .. of the n_host blocks of the whole input
        if (tp == nullptr || a.n_host <= 0 || a.n_host > kTpSelBlocks || a.mask_block0 < 0 ||
            a.mask_block0 + a.k / kBlockK > a.n_host || a.k_host < 0 || a.k_host > a.n_host)
          return BAS_ERR_INVALID_ARGUMENT;
        // its scores use the one region of the exchange area: every rank must have finished with the entry before
        // (i.e. the row-parallel call that ran with that entry's mask must be complete) - this entry has to
        // depend, directly or through other calls, on the last row-parallel call before it, which must lie
        // behind the previous sharded entry
        int prev_entry = -1, prev_row = -1;
        for (int q = c - 1; q >= 0; --q) {
          if (prev_row < 0 && calls[q].op == BAS_LIST_GEMM && calls[q].row_parallel != 0) prev_row = q;
          if (calls[q].op == BAS_LIST_SELECT && (calls[q].shape_flags & BAS_LIST_SELECT_SHARDED) != 0) {
            prev_entry = q;
            break;
          }
        }
        if (prev_entry >= 0) {
          if (prev_row < prev_entry) return BAS_ERR_INVALID_ARGUMENT;
          int d = a.depends_on;
          while (d > prev_row) d = calls[d].depends_on;
          if (d != prev_row) return BAS_ERR_INVALID_ARGUMENT;
        }
        ++n_sharded;
        if (a.n_host > sel_nb_max) sel_nb_max = a.n_host;
      } else if (a.n_host != 0 || a.mask_block0 != 0 || a.k_host < 0 || a.k_host > a.k / kBlockK) {
        return BAS_ERR_INVALID_ARGUMENT;
      }
      if (a.score_kind != BAS_SCORE_NORM && a.score_kind != BAS_SCORE_ENERGY) return BAS_ERR_INVALID_ARGUMENT;
      if (!list_aligned16(a.x_dev) || (a.ldx & 7) != 0) return BAS_ERR_INVALID_ARGUMENT;
      if (a.depends_on < -1 || a.depends_on >= c || a.row_parallel != 0 || a.mask_entry != 0) return BAS_ERR_INVALID_ARGUMENT;
      if (a.packed_dev != nullptr || a.y_dev != nullptr || a.ids_dev != nullptr || a.count_dev != nullptr ||
          a.bitmap_dev != nullptr || a.ids_out_dev != nullptr || a.n_ids_dev != nullptr || a.n != 0)
        return BAS_ERR_INVALID_ARGUMENT;
      if (a.batch > max_batch) max_batch = a.batch;
      if (a.k / kBlockK > sel_nb_max) sel_nb_max = a.k / kBlockK;
      ++n_sel;
      continue;
    }
    if (a.op != BAS_LIST_GEMM) return BAS_ERR_INVALID_ARGUMENT;
    ++n_gemm;
    if (a.x_dev == nullptr || a.packed_dev == nullptr || a.y_dev == nullptr) return BAS_ERR_INVALID_ARGUMENT;
    if ((a.shape_flags & ~(BAS_LIST_OUT_COMPACT | BAS_LIST_X_COMPACT)) != 0) return BAS_ERR_INVALID_ARGUMENT;
    const bool by_block = a.n_ids_dev != nullptr, x_compact = (a.shape_flags & BAS_LIST_X_COMPACT) != 0;
    if (by_block || x_compact) ++n_shaped;
    if (by_block) {
      if (a.n_host <= 0 || a.n_host > (a.n + 63) / 64 || a.row_parallel != 0) return BAS_ERR_INVALID_ARGUMENT;
    } else if (a.n_host != 0 || (a.shape_flags & BAS_LIST_OUT_COMPACT) != 0) {
      return BAS_ERR_INVALID_ARGUMENT;
    }
    if (x_compact && (a.row_parallel != 0 || a.mask_entry != 0 || a.bitmap_dev != nullptr || a.ids_dev == nullptr))
      return BAS_ERR_INVALID_ARGUMENT;          // compact X goes with an id list: its order is X's
    // the widths the caller's buffers must have: compact X holds k_host blocks, a compact Y n_host blocks
    const long long x_cols = x_compact ? (long long)a.k_host * kBlockK : (long long)a.k;
    const long long y_cols = (by_block && (a.shape_flags & BAS_LIST_OUT_COMPACT) != 0) ? (long long)a.n_host * 64 : (long long)a.n;
    if (a.batch <= 0 || a.k <= 0 || a.n <= 0 || a.k_host < 0 || a.ldx < x_cols || a.ldy < y_cols) return BAS_ERR_INVALID_ARGUMENT;
    if (a.batch > BAS_MAX_BATCH) return BAS_ERR_UNSUPPORTED;
    const int nb = (a.k + kBlockK - 1) / kBlockK;
    if (nb > BAS_LIST_MAX_BLOCKS) return BAS_ERR_UNSUPPORTED;
    if (a.mask_entry != 0) {
      // the mask comes from an earlier selection entry of the same X (same shape of the batch, same call waited
      // for), of which this call may cover a range of blocks
      const int en = a.mask_entry - 1;
      if (en < 0 || en >= c || calls[en].op != BAS_LIST_SELECT) return BAS_ERR_INVALID_ARGUMENT;
      if (a.ids_dev != nullptr || a.count_dev != nullptr || a.bitmap_dev != nullptr) return BAS_ERR_INVALID_ARGUMENT;
      if (calls[en].depends_on != a.depends_on || calls[en].batch != a.batch || (a.k % kBlockK) != 0) return BAS_ERR_INVALID_ARGUMENT;
      if ((calls[en].shape_flags & BAS_LIST_SELECT_SHARDED) != 0) {
        // the entry saw this rank's K-shard only: the call is the row-parallel one over that very shard
        if (a.row_parallel == 0 || a.mask_block0 != calls[en].mask_block0 || nb != calls[en].k / kBlockK || a.ids_out_dev != nullptr)
          return BAS_ERR_INVALID_ARGUMENT;
      } else if (a.mask_block0 < 0 || a.mask_block0 + nb > calls[en].k / kBlockK) {
        return BAS_ERR_INVALID_ARGUMENT;
      }
    } else {
      if (a.mask_block0 != 0 || a.ids_out_dev != nullptr) return BAS_ERR_INVALID_ARGUMENT;
      if (a.bitmap_dev == nullptr && a.ids_dev == nullptr && a.k_host > 0) return BAS_ERR_INVALID_ARGUMENT;
      if (a.bitmap_dev == nullptr && a.k_host > nb) return BAS_ERR_INVALID_ARGUMENT;
    }
    if (!list_aligned16(a.x_dev) || !list_aligned16(a.packed_dev) || (a.ldx & 7) != 0 || (a.k & 7) != 0)
      return BAS_ERR_INVALID_ARGUMENT;
    if (a.depends_on < -1 || a.depends_on >= c) return BAS_ERR_INVALID_ARGUMENT;
    if (a.row_parallel != 0) {
      // an exchange needs a connected group that holds this output, and - the two receive buffers alternate - the
      // exchange before it must be complete on every rank before this one starts: it has to depend on it
      if (tp == nullptr || a.row_parallel != 1 || a.batch > tp->max_batch || a.n > tp->n) return BAS_ERR_INVALID_ARGUMENT;
      int prev = -1;
      for (int q = c - 1; q >= 0 && prev < 0; --q)
        if (calls[q].row_parallel != 0) prev = q;
      if (prev >= 0) {
        int d = a.depends_on;
        while (d > prev) d = calls[d].depends_on;
        if (d != prev) return BAS_ERR_INVALID_ARGUMENT;
      }
    }
    if (a.batch > max_batch) max_batch = a.batch;
    if (nb > nb_max) nb_max = nb;
  }
  if (n_gemm == 0) return BAS_ERR_INVALID_ARGUMENT;
  const int bpad = (max_batch + 15) / 16 * 16;
  e = by_bpad(bpad, [](auto b) { return list_prepare_kernel<decltype(b)::value>(); });
  if (e != cudaSuccess) return record_cuda_error(e);

  // ---- cluster size and grid ----
  // One CTA per column range unless the caller asks for clusters: measured on the Llama-2-7B stack
  // (batch 16) the cluster modes, whose CTAs meet once per column tile to add their partials, run at a
  // third of the rate of independent CTAs, with or without dependencies between the calls.
  const int forced = (flags >> 8) & 7;
  const int cta_cap = ((flags >> 16) & 0xff) != 0 ? ((flags >> 16) & 0xff) : sm_count;
  if (forced != 0 && forced != 1 && forced != 2 && forced != 4) return BAS_ERR_INVALID_ARGUMENT;
  if (tp != nullptr) {
    if (forced > 1) return BAS_ERR_INVALID_ARGUMENT;           // the exchange is built for one CTA per range
    for (int q = 0; q < tp->world; ++q)
      if (tp->area[q] == nullptr) return BAS_ERR_INVALID_ARGUMENT;   // bas_tp_connect has not run
  }
  if ((n_sel > 0 || n_shaped > 0) && forced > 1) return BAS_ERR_UNSUPPORTED;   // selection entries, output blocks, compact X: one CTA per range only
  const int cluster = forced != 0 ? forced : 1;
  int n_clusters = by_bpad(bpad, [&](auto b) { return list_resident_clusters<decltype(b)::value>(cluster, kLSmemBudget, sm_count); });
  if (n_clusters > cta_cap / cluster) n_clusters = cta_cap / cluster;
  if (n_clusters <= 0) return BAS_ERR_UNSUPPORTED;

  // ---- per call: the clusters that take part, and the widest column tile of the list ----
  const int min_units = ((flags >> 24) & 0x3f) != 0 ? ((flags >> 24) & 0x3f) : 8;   // tuning knob
  std::vector<ListCallDev> host((size_t)n_calls);
  int off = 0, tw_max = 8, n_tp = 0, sel_seen = 0, sharded_seen = 0;
  for (int c = 0; c < n_calls; ++c) {
    const bas_list_call& a = calls[c];
    ListCallDev& d = host[(size_t)c];
    std::memset(&d, 0, sizeof(d));
    if (a.op == BAS_LIST_SELECT) {
      // one block per CTA and round where there are enough CTAs; `scores` holds the entry's number until the
      // device block exists
      d.nb = a.k / kBlockK;
      d.ranges = d.nb < n_clusters ? d.nb : n_clusters;
      d.units = d.ranges;
      d.range_off = (d.ranges < n_clusters) ? off : 0;
      if (d.ranges < n_clusters) off = (off + d.ranges) % n_clusters;
      d.packed = (const uint8_t*)a.x_dev;
      d.ids = (const int32_t*)(uintptr_t)sel_seen++;                                   // score array: its number for now
      d.count_dev = (const int32_t*)(uintptr_t)(unsigned long long)a.ldx;              // row stride of X
      d.bitmap = (const uint8_t*)(uintptr_t)(unsigned long long)(unsigned int)a.score_kind;   // high half: see below
      d.k_host = a.k_host;
      d.batch = a.batch;
      d.n = 0;
      d.tp_index = -1;
      d.dep = a.depends_on;
      if ((a.shape_flags & BAS_LIST_SELECT_SHARDED) != 0) {
        d.range_off |= kCallSharded;
        d.w_rows = a.mask_block0;         // first block of this rank's shard in the whole input
        d.out_compact = a.n_host;         // blocks of the whole input
        d.tp_index = sharded_seen++;      // the entry's number among the run's sharded entries
      }
      continue;
    }
    const bool by_block = a.n_ids_dev != nullptr, x_compact = (a.shape_flags & BAS_LIST_X_COMPACT) != 0;
    // (output blocks: the column space is the list of blocks, 64 columns each, and no range holds part of a block)
    const int npad = by_block ? a.n_host * 64 : padded_cols(a.n), units = npad / 8;
    int ranges = by_block ? a.n_host : units / min_units;      // no range narrower than min_units * 8 columns where the output allows
    if (ranges < 1) ranges = 1;
    if (ranges > n_clusters) ranges = n_clusters;
    // widest range of this call, its column tiles
    const int wmax = by_block ? ((a.n_host + ranges - 1) / ranges) * 64 : ((units + ranges - 1) / ranges) * 8;
    const int n_sub = by_block ? wmax / 64 : (wmax + kTileN - 1) / kTileN;
    if (n_sub > 16) return BAS_ERR_UNSUPPORTED;
    const int tw = by_block ? 64 : ((wmax + n_sub - 1) / n_sub + 7) & ~7;
    if (tw > tw_max) tw_max = tw;
    d.packed = (const uint8_t*)a.packed_dev;
    d.ids = a.bitmap_dev != nullptr ? nullptr : a.ids_dev;
    d.count_dev = a.bitmap_dev != nullptr ? nullptr : a.count_dev;
    d.bitmap = a.bitmap_dev;
    d.y = (__half*)a.y_dev;
    d.ldy = (long long)a.ldy;
    d.nb = (a.k + kBlockK - 1) / kBlockK;
    d.k_host = a.k_host > d.nb ? d.nb : a.k_host;
    if (a.mask_entry != 0) {
      const ListCallDev& en = host[(size_t)(a.mask_entry - 1)];
      d.k_host = -a.mask_entry;                // = -(entry + 1)
      d.ids = en.ids;                          // the entry's score array (still its number)
      d.count_dev = (const int32_t*)(uintptr_t)(unsigned long long)(unsigned int)
                    ((en.range_off & kCallSharded) != 0 ? en.out_compact : en.nb);
      d.bitmap = (const uint8_t*)(uintptr_t)(unsigned long long)(unsigned int)a.mask_block0;
      d.ids_out = a.ids_out_dev;
    }
    d.batch = a.batch;
    d.n = a.n;
    d.units = units;
    d.ranges = ranges;
    d.range_off = ((ranges < n_clusters) ? off : 0) | (by_block ? kCall2d : 0) | (x_compact ? kCallXCompact : 0);
    if (a.mask_entry != 0 && (host[(size_t)(a.mask_entry - 1)].range_off & kCallSharded) != 0)
      d.range_off |= kCallSharded;        // the entry saw a K-shard: this call has the verdicts of its own blocks only
    if (ranges < n_clusters) off = (off + ranges) % n_clusters;
    d.n_ids = a.n_ids_dev;
    d.w_rows = padded_cols(a.n);
    d.out_compact = (by_block && (a.shape_flags & BAS_LIST_OUT_COMPACT) != 0) ? 1 : 0;
    d.tp_index = a.row_parallel != 0 ? n_tp++ : -1;
    d.dep = a.depends_on;
    d.dep_contrib = a.depends_on >= 0 ? (unsigned int)(host[(size_t)a.depends_on].ranges * cluster) : 0u;
    // X[batch, K]: inner dimension K, box {64 channels, bpad rows}, 128-byte swizzle, zeros out of range
    auto encode = (PFN_cuTensorMapEncodeTiled_v12000)tensor_map_encoder();
    if (encode == nullptr) return record_cuda_error(cudaErrorNotSupported);
    const cuuint64_t gdim[2] = {(cuuint64_t)(x_compact ? (long long)a.k_host * kBlockK : (long long)a.k), (cuuint64_t)a.batch};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)bpad};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(&d.xmap, (flags & BAS_GEMM_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                              2, const_cast<void*>(a.x_dev), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return record_cuda_error(cudaErrorInvalidValue);
  }

  // ---- ring: slots of one weight tile + one activation tile ----
  const int wslot = (int)round_up((size_t)tw_max * kRowBytes, 1024);
  const size_t tile_bytes = (size_t)wslot + (size_t)bpad * 128;
  const size_t fixed = list_fixed_smem(n_calls, nb_max, cluster, bpad);
  const size_t pad = (size_t)kLMmaSpanBytes > (size_t)wslot ? (size_t)kLMmaSpanBytes - (size_t)wslot : 0;
  if (fixed + pad + 2 * tile_bytes > kLSmemBudget) return BAS_ERR_UNSUPPORTED;
  int slots = (int)((kLSmemBudget - fixed - pad) / tile_bytes);
  if (slots > kMaxStages) slots = kMaxStages;
  if (const char* cap = std::getenv("BAS_LIST_MAX_SLOTS")) {   // tuning knob
    const int v = std::atoi(cap);
    if (v >= 2 && v < slots) slots = v;
  }
  int pairs = (flags >> 12) & 7;
  if (pairs < 2 || pairs > kLProducers || slots / pairs == 0) {
    pairs = 0;
    int best = 2;
    for (int cnd = kLProducers; cnd >= 2; --cnd) {
      const int kept = slots / cnd * cnd;
      if (kept * 4 >= slots * 3) {
        pairs = cnd;
        break;
      }
      if (kept > slots / best * best) best = cnd;
    }
    if (pairs == 0) pairs = best;
  }
  // MMA-issuing warps: as many as tensor memory has accumulators for, a multiple of the copy warps;
  // the ring is a multiple of both, so that every warp always meets the same slots
  int issuers = (2 * kLIssuers * bpad <= 512) ? kLIssuers : 4;
  while (issuers > pairs && (issuers % pairs != 0 || slots / issuers == 0)) issuers -= 1;
  if (issuers < pairs || issuers % pairs != 0) issuers = pairs;
  slots = slots / issuers * issuers;
  if (slots < 2) return BAS_ERR_UNSUPPORTED;

  // A selection entry is reported by every copy warp that scored a block of it (block j: range j % ranges,
  // warp (j / ranges) % pairs): min(blocks, ranges * pairs) reports.  Whoever waits for an entry expects that many.
  for (int c = 0; c < n_calls; ++c) {
    ListCallDev& d = host[(size_t)c];
    auto reports = [&](int q) -> unsigned int {
      const ListCallDev& t = host[(size_t)q];
      if (calls[q].op != BAS_LIST_SELECT) return (unsigned int)(t.ranges * cluster);
      return (unsigned int)(t.nb < t.ranges * pairs ? t.nb : t.ranges * pairs);
    };
    if (d.dep >= 0) d.dep_contrib = reports(d.dep);
    if (calls[c].op == BAS_LIST_SELECT && d.dep >= 0)       // high half of the `bitmap` slot
      d.bitmap = (const uint8_t*)((uintptr_t)d.bitmap | ((uintptr_t)d.dep_contrib << 32));
    if (calls[c].op == BAS_LIST_SELECT)                     // high half of the `count_dev` slot: its own reports
      d.count_dev = (const int32_t*)((uintptr_t)d.count_dev | ((uintptr_t)reports(c) << 32));
  }

  bas_list* l = new (std::nothrow) bas_list();
  if (l == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  l->n_calls = n_calls;
  l->bpad = bpad;
  l->sm_count = sm_count;
  l->smem = fixed + pad + (size_t)slots * tile_bytes;
  const size_t counters_off = 256;
  const size_t desc_off = counters_off + round_up((size_t)n_calls * 4, 256);
  const size_t scores_off = round_up(desc_off + sizeof(ListCallDev) * (size_t)n_calls, 256);
  // per entry: kSelReplicas copies of its scores (double[rep_words]) and then as many copies of its verdict
  // words (unsigned[rep_words]: run number << 1 | kept), which start as zero - the number of no run
  const size_t rep_words = round_up((size_t)sel_nb_max * sizeof(double), 256) / sizeof(double);
  const size_t scores_stride = rep_words * kSelReplicas * (sizeof(double) + sizeof(unsigned int));
  l->dev_bytes = scores_off + scores_stride * (size_t)n_sel;
  e = cudaMalloc(&l->dev_block, l->dev_bytes);
  if (e == cudaSuccess) e = cudaMemset(l->dev_block, 0, desc_off);
  if (e == cudaSuccess && n_sel > 0) e = cudaMemset((uint8_t*)l->dev_block + scores_off, 0, scores_stride * (size_t)n_sel);
  l->sel_off = scores_off;
  for (int c = 0; c < n_calls && e == cudaSuccess; ++c)     // the entries' score arrays, now that they have an address
    if (calls[c].op == BAS_LIST_SELECT || calls[c].mask_entry != 0)
      host[(size_t)c].ids = (const int32_t*)((uint8_t*)l->dev_block + scores_off + scores_stride * (size_t)(uintptr_t)host[(size_t)c].ids);
  if (e == cudaSuccess)
    e = cudaMemcpy((uint8_t*)l->dev_block + desc_off, host.data(), sizeof(ListCallDev) * (size_t)n_calls, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (l->dev_block != nullptr) cudaFree(l->dev_block);
    delete l;
    return record_cuda_error(e);
  }
  ListParams& p = l->params;
  p.calls = (const ListCallDev*)((uint8_t*)l->dev_block + desc_off);
  p.n_calls = n_calls;
  p.hdr = (ListHeaderDev*)l->dev_block;
  p.done = (unsigned int*)((uint8_t*)l->dev_block + counters_off);
  p.cluster = cluster;
  p.n_clusters = n_clusters;
  p.stages = slots;
  p.pairs = pairs;
  p.issuers = issuers;
  p.wslot = wslot;
  p.nb_max = nb_max;
  p.sel_nb_max = sel_nb_max;
  p.extended = (n_sel > 0 || n_shaped > 0) ? 1 : 0;
  p.sel_rep_stride = (int)rep_words;
  p.bf16 = (flags & BAS_GEMM_BF16) != 0 ? 1 : 0;
  p.stall_call = -1;
  p.wait_cycles = wait_cycles_now();
  p.tp = TpExchange{};
  p.n_tp_calls = n_tp;
  p.n_sharded = n_sharded;
  if (tp != nullptr && n_tp > 0) {
    p.tp.world = tp->world;
    p.tp.rank = tp->rank;
    p.tp.ldp = tp->npad;
    p.tp.src_words = (long long)tp->max_batch * tp->npad;
    p.tp.own = tp->area[tp->rank];
    p.tp.sel_words = (long long)((tp->bytes - kTpSelBytes) / 8);
    for (int q = 0; q < tp->world; ++q) p.tp.area[q] = tp->area[q];
  }
#ifdef BAS_TRACE
  p.trace = nullptr;
  p.trace_cta = 0;
  // [0, CALLS): the last stamp of each event over the CTAs; [CALLS, 2 CALLS): the first (kept by atomicMin, so it starts at all ones)
  if (cudaMalloc(&p.trace, sizeof(long long) * 2 * BAS_LTRACE_CALLS * BAS_LTRACE_EVENTS) == cudaSuccess)
    cudaMemset(p.trace, 0, sizeof(long long) * 2 * BAS_LTRACE_CALLS * BAS_LTRACE_EVENTS);
#endif
  *out = l;
  return BAS_OK;
}

BAS_API int bas_list_run(bas_list* l, void* stream) {
  if (l == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  count_launch();
  const cudaError_t e = by_bpad(l->bpad, [&](auto b) {
    return list_launch<decltype(b)::value>(l->params, l->smem, (cudaStream_t)stream);
  });
  return e == cudaSuccess ? BAS_OK : record_cuda_error(e);
}

BAS_API int bas_list_read_status(bas_list* l, unsigned int* flags_out, void* stream) {
  if (l == nullptr || flags_out == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(flags_out, &l->params.hdr->status, sizeof(unsigned int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(&l->params.hdr->status, 0, sizeof(unsigned int), s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  return e == cudaSuccess ? BAS_OK : record_cuda_error(e);
}

BAS_API int bas_list_reset(bas_list* l) {
  if (l == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemset(l->dev_block, 0, (size_t)((const uint8_t*)l->params.calls - (const uint8_t*)l->dev_block));
  // the run number starts again: verdicts of earlier runs must not pass for those of the runs to come
  if (e == cudaSuccess && l->dev_bytes > l->sel_off) e = cudaMemset((uint8_t*)l->dev_block + l->sel_off, 0, l->dev_bytes - l->sel_off);
  return e == cudaSuccess ? BAS_OK : record_cuda_error(e);
}

BAS_API int bas_list_set_wait(bas_list* l, double wait_ms, int never_ready_call) {
  if (l == nullptr || !(wait_ms > 0.0) || wait_ms > 10000.0 || never_ready_call < -1 || never_ready_call >= l->n_calls)
    return BAS_ERR_INVALID_ARGUMENT;
  l->params.wait_cycles = (long long)(wait_ms * 2.0e6);   // clock64 ticks at about 2 GHz
  l->params.stall_call = never_ready_call;
  return BAS_OK;
}

BAS_API int bas_list_info(const bas_list* l, int* ctas, int* cluster, int* slots, int* pairs) {
  if (l == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  if (ctas != nullptr) *ctas = l->params.n_clusters * l->params.cluster;
  if (cluster != nullptr) *cluster = l->params.cluster;
  if (slots != nullptr) *slots = l->params.stages;
  if (pairs != nullptr) *pairs = l->params.pairs;
  return BAS_OK;
}

#ifdef BAS_TRACE
// Diagnostic build: copies the event stamps ([call][event], nanoseconds of the global timer) to the host,
// clears them and chooses the CTA that stamps the next runs.
BAS_API int bas_list_debug_trace(bas_list* l, long long* out, int n, int next_cta) {
  if (l == nullptr || l->params.trace == nullptr) return 1;
  const size_t half = (size_t)BAS_LTRACE_CALLS * BAS_LTRACE_EVENTS, total = 2 * half;
  const size_t cnt = (size_t)n < total ? (size_t)n : total;
  cudaError_t e = cudaMemcpy(out, l->params.trace, sizeof(long long) * cnt, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemset(l->params.trace, 0, sizeof(long long) * total);
  l->params.trace_cta = next_cta;
  return e == cudaSuccess ? 0 : 4;
}
#endif

BAS_API void bas_list_destroy(bas_list* l) {
  if (l == nullptr) return;
  if (l->dev_block != nullptr) cudaFree(l->dev_block);
  delete l;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// host-buffer operator for a whole step (bas_step_*): the calls of one decode step whose activations
// live in host memory, as ONE unit of submission - all uploads, the mask selections, one list
// launch for all contractions, all downloads - with several steps in flight on streams of their own.
// ---------------------------------------------------------------------------------------------
struct bas_step {
  struct Call {
    int n, k, nb, batch, n_keep, score_kind;
    long long ldx;
    uint8_t* packed;         // owned by the step unless shared with an earlier call of the same weight
    size_t x_off, y_off;     // element offsets into a slot's device X / Y blocks
    size_t ids_off;          // int32 offset into a slot's id block
  };
  struct Slot {
    cudaStream_t stream = nullptr;
    __half* x_dev = nullptr;
    __half* y_dev = nullptr;
    uint8_t* small_dev = nullptr;     // [ids of all calls][pad] ; the list's status word is copied beside it
    uint8_t* small_pin = nullptr;
    uint8_t* sel_ws = nullptr;        // one selection workspace per call (the calls' selections run side by side)
    cudaStream_t aux[3] = {nullptr, nullptr, nullptr};   // branches beside `stream` for uploads + selections
    cudaEvent_t fork = nullptr, join[3] = {nullptr, nullptr, nullptr};
    bas_list* list = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<const void*> key;     // host pointers the graph was captured with
    std::vector<int32_t*> ids_out;
    bool pending = false, graph_failed = false;
  };
  std::vector<Call> calls;
  std::vector<uint8_t*> owned_packed;
  std::vector<Slot> slots;
  size_t x_elems = 0, y_elems = 0, ids_count = 0, small_bytes = 0, sel_ws_bytes = 0;
  unsigned long long submitted = 0, waited = 0;
};

namespace {

bool step_is_pinned(const void* ptr) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeHost;
}

// The stream work of one step: uploads, selections, the list launch, downloads.  Nothing is waited for.
int step_enqueue(bas_step* st, bas_step::Slot& sl, const void* const* x_host, void* const* y_host) {
  cudaStream_t s = sl.stream;
  // Upload and selection of call c run on branch c % branches: a call's selection starts as soon as its
  // own X has arrived, and the calls' selections (a few microseconds of latency each) overlap.
  const int branches = (int)std::min<size_t>(st->calls.size(), 4);
  cudaError_t e = cudaEventRecord(sl.fork, s);
  for (int i = 1; i < branches && e == cudaSuccess; ++i) e = cudaStreamWaitEvent(sl.aux[i - 1], sl.fork, 0);
  if (e != cudaSuccess) return record_cuda_error(e);
  int32_t* ids_base = (int32_t*)sl.small_dev;
  for (size_t c = 0; c < st->calls.size(); ++c) {
    const bas_step::Call& a = st->calls[c];
    cudaStream_t bs = (c % branches == 0) ? s : sl.aux[c % branches - 1];
    const size_t row = (size_t)a.k * 2;
    if ((size_t)a.ldx * 2 == row)      // rows are contiguous on both sides: one plain copy
      e = cudaMemcpyAsync(sl.x_dev + a.x_off, x_host[c], row * (size_t)a.batch, cudaMemcpyHostToDevice, bs);
    else
      e = cudaMemcpy2DAsync(sl.x_dev + a.x_off, (size_t)a.ldx * 2, x_host[c], row, row, (size_t)a.batch, cudaMemcpyHostToDevice, bs);
    if (e != cudaSuccess) return record_cuda_error(e);
    // count goes to the last word of the call's id block (nb + 1 words per call)
    const int rc = bas_select_topk(sl.x_dev + a.x_off, a.ldx, a.batch, a.k, a.n_keep, a.score_kind, ids_base + a.ids_off,
                                   ids_base + a.ids_off + a.nb, nullptr, nullptr, sl.sel_ws + c * st->sel_ws_bytes,
                                   st->sel_ws_bytes, bs);
    if (rc != BAS_OK) return rc;
  }
  for (int i = 1; i < branches; ++i) {
    e = cudaEventRecord(sl.join[i - 1], sl.aux[i - 1]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, sl.join[i - 1], 0);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  int rc = bas_list_run(sl.list, s);
  if (rc != BAS_OK) return rc;
  for (size_t c = 0; c < st->calls.size(); ++c) {
    const bas_step::Call& a = st->calls[c];
    cudaError_t e = cudaMemcpyAsync(y_host[c], sl.y_dev + a.y_off, (size_t)a.batch * a.n * 2, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  // the ids of every call and, behind them, the list's status word: one block, one copy
  e = cudaMemcpyAsync(sl.small_dev + st->ids_count * 4, &sl.list->params.hdr->status, sizeof(unsigned int),
                                  cudaMemcpyDeviceToDevice, s);
  if (e == cudaSuccess) e = cudaMemcpyAsync(sl.small_pin, sl.small_dev, st->small_bytes, cudaMemcpyDeviceToHost, s);
  return e == cudaSuccess ? BAS_OK : record_cuda_error(e);
}

void step_free(bas_step* st) {
  if (st == nullptr) return;
  for (auto& sl : st->slots) {
    if (sl.stream != nullptr) cudaStreamSynchronize(sl.stream);
    if (sl.exec != nullptr) cudaGraphExecDestroy(sl.exec);
    if (sl.list != nullptr) bas_list_destroy(sl.list);
    if (sl.x_dev != nullptr) cudaFree(sl.x_dev);
    if (sl.y_dev != nullptr) cudaFree(sl.y_dev);
    if (sl.small_dev != nullptr) cudaFree(sl.small_dev);
    if (sl.sel_ws != nullptr) cudaFree(sl.sel_ws);
    if (sl.small_pin != nullptr) cudaFreeHost(sl.small_pin);
    for (int i = 0; i < 3; ++i) {
      if (sl.aux[i] != nullptr) cudaStreamDestroy(sl.aux[i]);
      if (sl.join[i] != nullptr) cudaEventDestroy(sl.join[i]);
    }
    if (sl.fork != nullptr) cudaEventDestroy(sl.fork);
    if (sl.stream != nullptr) cudaStreamDestroy(sl.stream);
  }
  for (uint8_t* ptr : st->owned_packed) cudaFree(ptr);
  delete st;
}

}  // namespace

extern "C" {

BAS_API int bas_step_create(bas_step** out, const bas_step_call* calls, int n_calls, int depth) {
  if (out == nullptr || calls == nullptr || n_calls <= 0 || n_calls > 1024 || depth < 1 || depth > 8) return BAS_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  bas_step* st = new (std::nothrow) bas_step();
  if (st == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  cudaError_t e = cudaSuccess;
  int rc = BAS_OK;
  int k_max = 0;
  // ---- weights: packed once; calls that name the same host weight share the pack ----
  for (int c = 0; c < n_calls && rc == BAS_OK && e == cudaSuccess; ++c) {
    const bas_step_call& in = calls[c];
    if (in.w_host == nullptr || in.n <= 0 || in.k < kBlockK || in.batch <= 0 || in.batch > BAS_MAX_BATCH || in.n_keep < 1 ||
        in.n_keep > in.k / kBlockK || (in.score_kind != BAS_SCORE_NORM && in.score_kind != BAS_SCORE_ENERGY)) {
      rc = BAS_ERR_INVALID_ARGUMENT;
      break;
    }
    bas_step::Call a;
    a.n = in.n;
    a.k = in.k;
    a.nb = (in.k + kBlockK - 1) / kBlockK;
    a.batch = in.batch;
    a.n_keep = in.n_keep;
    a.score_kind = in.score_kind;
    a.ldx = ((long long)in.k + 7) / 8 * 8;
    a.packed = nullptr;
    for (int p = 0; p < c; ++p)
      if (calls[p].w_host == in.w_host && calls[p].n == in.n && calls[p].k == in.k) a.packed = st->calls[(size_t)p].packed;
    if (a.packed == nullptr) {
      __half* w_dev = nullptr;
      e = cudaMalloc(&w_dev, (size_t)in.n * in.k * 2);
      if (e == cudaSuccess) e = cudaMalloc(&a.packed, bas_packed_weight_bytes(in.n, in.k));
      if (e == cudaSuccess) st->owned_packed.push_back(a.packed);
      if (e == cudaSuccess) e = cudaMemcpy(w_dev, in.w_host, (size_t)in.n * in.k * 2, cudaMemcpyHostToDevice);
      if (e == cudaSuccess) rc = bas_pack_weight(w_dev, in.n, in.k, in.k, a.packed, nullptr);
      if (e == cudaSuccess) e = cudaDeviceSynchronize();
      if (w_dev != nullptr) cudaFree(w_dev);
    }
    a.x_off = st->x_elems;
    a.y_off = st->y_elems;
    a.ids_off = st->ids_count;
    st->x_elems += (size_t)a.batch * (size_t)a.ldx;
    st->y_elems += (size_t)a.batch * (size_t)a.n;
    st->ids_count += (size_t)a.nb + 1;
    if (in.k > k_max) k_max = in.k;
    st->calls.push_back(a);
  }
  st->small_bytes = st->ids_count * 4 + 16;
  st->sel_ws_bytes = (bas_select_workspace_bytes(k_max) + 255) / 256 * 256;
  // ---- slots: device blocks, a stream and a list of the step's contractions each ----
  st->slots.resize((size_t)depth);
  for (auto& sl : st->slots) {
    if (rc != BAS_OK || e != cudaSuccess) break;
    e = cudaStreamCreateWithFlags(&sl.stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&sl.x_dev, st->x_elems * 2);
    if (e == cudaSuccess) e = cudaMemset(sl.x_dev, 0, st->x_elems * 2);          // row padding stays zero
    if (e == cudaSuccess) e = cudaMalloc(&sl.y_dev, st->y_elems * 2);
    if (e == cudaSuccess) e = cudaMalloc(&sl.small_dev, st->small_bytes);
    if (e == cudaSuccess) e = cudaMemset(sl.small_dev, 0, st->small_bytes);
    if (e == cudaSuccess) e = cudaMallocHost(&sl.small_pin, st->small_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&sl.sel_ws, st->sel_ws_bytes * (size_t)n_calls);
    if (e == cudaSuccess) e = cudaMemset(sl.sel_ws, 0, st->sel_ws_bytes * (size_t)n_calls);
    for (int i = 0; i < 3 && e == cudaSuccess; ++i) {
      e = cudaStreamCreateWithFlags(&sl.aux[i], cudaStreamNonBlocking);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&sl.join[i], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&sl.fork, cudaEventDisableTiming);
    if (e != cudaSuccess) break;
    std::vector<bas_list_call> lc((size_t)n_calls);
    for (int c = 0; c < n_calls; ++c) {
      const bas_step::Call& a = st->calls[(size_t)c];
      bas_list_call& d = lc[(size_t)c];
      std::memset(&d, 0, sizeof(d));
      d.x_dev = sl.x_dev + a.x_off;
      d.ldx = a.ldx;
      d.packed_dev = a.packed;
      d.ids_dev = (const int32_t*)sl.small_dev + a.ids_off;
      d.k_host = a.n_keep;
      d.batch = a.batch;
      d.k = (int)a.ldx;
      d.n = a.n;
      d.y_dev = sl.y_dev + a.y_off;
      d.ldy = a.n;
      d.depends_on = -1;
    }
    rc = bas_list_create(&sl.list, lc.data(), n_calls, 16 << 24);   // 128-column ranges: mixed batch sizes up to 64
  }
  if (rc == BAS_OK && e == cudaSuccess) e = cudaDeviceSynchronize();
  if (rc != BAS_OK || e != cudaSuccess) {
    step_free(st);
    return rc != BAS_OK ? rc : record_cuda_error(e);
  }
  *out = st;
  return BAS_OK;
}

BAS_API int bas_step_submit(bas_step* st, const void* const* x_host, void* const* y_host, int32_t* const* ids_host_out) {
  if (st == nullptr || x_host == nullptr || y_host == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  bas_step::Slot& sl = st->slots[(size_t)(st->submitted % st->slots.size())];
  if (sl.pending) return BAS_ERR_INVALID_ARGUMENT;   // every slot is in flight: wait first
  const size_t n = st->calls.size();
  std::vector<const void*> key;
  key.reserve(2 * n);
  bool pinned = true;
  for (size_t c = 0; c < n; ++c) {
    if (x_host[c] == nullptr || y_host[c] == nullptr) return BAS_ERR_INVALID_ARGUMENT;
    key.push_back(x_host[c]);
    key.push_back(y_host[c]);
  }
  int rc;
  if (sl.exec != nullptr && sl.key == key) {
    const cudaError_t e = cudaGraphLaunch(sl.exec, sl.stream);
    rc = e == cudaSuccess ? BAS_OK : record_cuda_error(e);
  } else {
    // A step that recurs with the same page-locked buffers is captured on its second occurrence and
    // replayed from then on (one graph launch instead of a dozen stream calls).
    for (size_t c = 0; c < 2 * n && pinned; ++c) pinned = step_is_pinned(key[c]);
    const bool capture = pinned && !sl.graph_failed && sl.key == key && sl.exec == nullptr;
    if (sl.key != key && sl.exec != nullptr) {
      cudaGraphExecDestroy(sl.exec);
      sl.exec = nullptr;
    }
    sl.key = key;
    if (capture) {
      cudaGraph_t graph = nullptr;
      cudaError_t e = cudaStreamBeginCapture(sl.stream, cudaStreamCaptureModeThreadLocal);
      if (e == cudaSuccess) {
        rc = step_enqueue(st, sl, x_host, y_host);
        e = cudaStreamEndCapture(sl.stream, &graph);
        if (rc == BAS_OK && e == cudaSuccess && graph != nullptr) e = cudaGraphInstantiate(&sl.exec, graph, 0);
        else if (e == cudaSuccess) e = cudaErrorUnknown;
        if (graph != nullptr) cudaGraphDestroy(graph);
      }
      if (e != cudaSuccess || sl.exec == nullptr) {
        (void)cudaGetLastError();
        sl.exec = nullptr;
        sl.graph_failed = true;
        rc = step_enqueue(st, sl, x_host, y_host);
      } else {
        e = cudaGraphLaunch(sl.exec, sl.stream);
        rc = e == cudaSuccess ? BAS_OK : record_cuda_error(e);
      }
    } else {
      rc = step_enqueue(st, sl, x_host, y_host);
    }
  }
  if (rc != BAS_OK) return rc;
  sl.ids_out.assign(n, nullptr);
  if (ids_host_out != nullptr)
    for (size_t c = 0; c < n; ++c) sl.ids_out[c] = ids_host_out[c];
  sl.pending = true;
  ++st->submitted;
  return BAS_OK;
}

BAS_API int bas_step_wait(bas_step* st) {
  if (st == nullptr || st->waited >= st->submitted) return BAS_ERR_INVALID_ARGUMENT;
  bas_step::Slot& sl = st->slots[(size_t)(st->waited % st->slots.size())];
  ++st->waited;
  sl.pending = false;
  const cudaError_t e = cudaStreamSynchronize(sl.stream);
  if (e != cudaSuccess) return record_cuda_error(e);
  const int32_t* ids = (const int32_t*)sl.small_pin;
  for (size_t c = 0; c < st->calls.size(); ++c)
    if (sl.ids_out[c] != nullptr) std::memcpy(sl.ids_out[c], ids + st->calls[c].ids_off, sizeof(int32_t) * (size_t)st->calls[c].n_keep);
  unsigned int flags = 0;
  std::memcpy(&flags, sl.small_pin + st->ids_count * 4, sizeof(flags));
  if (flags != 0) {
    cudaMemsetAsync(&sl.list->params.hdr->status, 0, sizeof(unsigned int), sl.stream);
    return BAS_ERR_DEVICE_FLAG;
  }
  return BAS_OK;
}

BAS_API void bas_step_destroy(bas_step* st) { step_free(st); }

}  // extern "C"
