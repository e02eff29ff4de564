// Shared device helpers: mbarrier, bulk-async copies, tcgen05 and cluster wrappers, and the column
// split used by both contraction kernels.  sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bas.h"
#include "bas_trace.cuh"

namespace bas {

constexpr int kBlockK = BAS_BLOCK_K;                 // channels per activation block
constexpr int kTileN = BAS_TILE_N;                   // widest column sub-tile one pass handles
constexpr int kRowBytes = kBlockK * 2;               // one output column's 64 fp16 weights of a block
constexpr int kMaxStages = 32;                       // ring slots (mbarrier arrays are sized for it)
constexpr long long kWaitCycles = 2000000000LL;      // bound of every barrier wait, about one second
constexpr size_t kWsBytes = 256;                     // workspace: [0,4) status word, rest reserved

// Column split: the (padded) output columns are cut, in units of 8 columns, into `ranges` contiguous
// ranges of near-equal width; one CTA (or one cluster of CTAs that split the active blocks among
// themselves) owns a range and needs no other CTA's data to finish it.
__host__ __device__ __forceinline__ int col_begin(int range, int units, int ranges) {
  return (int)((long long)range * units / ranges) * 8;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Adds to the pending byte count of the current phase without arriving.
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking look at a barrier (diagnostics).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the wait ran out or another role of this CTA already gave up
// (*abort_flag != 0); the caller then records BAS_DEV_WAIT_EXPIRED and leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag != 0 || clock64() - t0 > kWaitCycles) return false;
  }
  return true;
}

// The same with the bound given by the caller (kernels whose wait limit is a launch parameter).
__device__ __forceinline__ bool mbar_wait_for(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long limit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag != 0 || clock64() - t0 > limit) return false;
  }
  return true;
}
// Wait on a barrier of this CTA on which threads of OTHER CTAs of the cluster arrive (release at
// cluster scope): the acquire makes what they wrote into this CTA's shared memory visible.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster_for(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                      long long limit) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait_cluster(bar, parity)) {
    if (*abort_flag != 0 || clock64() - t0 > limit) return false;
  }
  return true;
}
// Arrive on a barrier that lives in the shared memory of a CTA of this cluster (address from
// dsmem_addr); releases, at cluster scope, what this thread wrote (and observed) before.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
// Orders this thread's generic-proxy accesses (plain loads and stores, also those it has observed
// through an acquire) against its asynchronous-proxy accesses (bulk / tensor copies), all state spaces.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// Completion counters in global memory that CTAs of one grid hand work over through.
__device__ __forceinline__ unsigned int ld_relaxed_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add_u32(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Arrival counter in shared memory: orders, at CTA scope, what the arriving thread wrote (and
// observed) before against what the thread that reads the count does afterwards.
__device__ __forceinline__ unsigned int atom_add_acq_rel_cta_shared_u32(unsigned int* p, unsigned int v) {
  unsigned int old;
  asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(p)), "r"(v) : "memory");
  return old;
}
// Shared-memory word one warp publishes to the other warps of its CTA.
__device__ __forceinline__ void st_release_cta_shared_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_cta_shared_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------------
// bulk asynchronous copies (TMA unit), completion counted in bytes on an mbarrier
// ---------------------------------------------------------------------------------------------
// 1-D: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(__cvta_generic_to_global(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// L2 eviction policy for the small operands that every CTA and the next call re-read (activations,
// id lists): evict-last, so that the weights streaming past do not push them out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ int ld_nc_keep_s32(const int32_t* p, uint64_t policy) {
  int v;
  asm volatile("ld.global.nc.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ unsigned int ld_nc_keep_u8(const uint8_t* p, uint64_t policy) {
  unsigned int v;
  asm volatile("ld.global.nc.L2::cache_hint.u8 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], "
      "[%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// 2-D tiled load through a tensor map; x (innermost coordinate) times the element size must be a
// multiple of 16 bytes.  Out-of-range elements arrive as zeros and still count towards the bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: tensor memory and 5th-generation tensor-core MMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; fp16 operands, fp32 accumulate.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 lanes x 16 consecutive fp32 columns: thread i of the warp receives lane (base + i).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes (64 fp16) and
// which is stored with the 128-byte swizzle: 8-row groups of 1024 bytes (stride-byte-offset 1024),
// leading-byte-offset field 1 (unused for swizzled K-major), descriptor version 1, layout type 2.
// The tile base must be 1024-byte aligned; advancing along K by 16 elements adds 32 bytes to the
// start address.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor: fp32 accumulator, fp16 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute
// may start while the previous kernel of the stream is still draining.  Everything before
// pdl_wait() must touch only this CTA's own shared/tensor memory (or data the previous kernel
// cannot be writing); pdl_wait() returns once the previous grid has completed and its writes are
// visible.  pdl_launch_dependents() lets the next kernel of the stream begin its own preamble.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Thread-block clusters: rank, barrier and distributed shared memory
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of all CTAs of the cluster; orders shared-memory writes before it against reads after it.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void dsmem_st_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void dsmem_st_v4_f32(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void dsmem_st_f64(uint32_t cluster_addr, double v) {
  asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(cluster_addr), "d"(v) : "memory");
}
__device__ __forceinline__ float dsmem_ld_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------------
// Active-set staging by ONE warp (all 32 lanes call it): builds the compact 16-bit list of valid
// block ids in shared memory, in input order.
//  * id list: an entry outside [0, nb) is dropped and flagged in the status word;
//  * byte map: the non-zero positions in ascending order.
// Returns the list length.  The caller publishes it to the other warps.
// ---------------------------------------------------------------------------------------------
// One batch of up to 256 source entries (ids or byte-map bytes), eight per lane, loaded together so
// that their latencies overlap.
__device__ __forceinline__ void warp_load_id_batch(const int32_t* __restrict__ ids, const uint8_t* __restrict__ bitmap,
                                                   int n_src, int base0, int lane, int (&raw)[8]) {
  const uint64_t keep = l2_policy_evict_last();   // the list is read by every CTA, and small
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int e = base0 + u * 32 + lane;
    raw[u] = 0;
    if (e < n_src) raw[u] = (bitmap != nullptr) ? (int)ld_nc_keep_u8(bitmap + e, keep) : ld_nc_keep_s32(ids + e, keep);
  }
}

// With `have_first`, `first` is the batch at offset 0 already loaded by the caller with
// warp_load_id_batch and the same n_src: a kernel issues it before its set-up work when the list is
// known not to depend on the kernel running before it.
__device__ __forceinline__ int warp_stage_ids(const int32_t* __restrict__ ids, const int32_t* __restrict__ count_dev,
                                              int k_host, const uint8_t* __restrict__ bitmap, int nb,
                                              uint16_t* __restrict__ s_ids, unsigned int* __restrict__ status,
                                              int lane, bool have_first, const int (&first)[8],
                                              bool report_bad = (blockIdx.x == 0)) {
  int n_src = nb;
  if (bitmap == nullptr) {
    n_src = k_host;
    if (count_dev != nullptr) n_src = min(max(__ldg(count_dev), 0), k_host);
  }
  int off = 0;
  bool bad = false;
  for (int base0 = 0; base0 < n_src; base0 += 256) {
    int raw[8];
    if (base0 == 0 && have_first) {
#pragma unroll
      for (int u = 0; u < 8; ++u) raw[u] = first[u];
    } else {
      warp_load_id_batch(ids, bitmap, n_src, base0, lane, raw);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int e = base0 + u * 32 + lane;
      if (base0 + u * 32 < n_src) {     // warp-uniform
        int id = e;
        bool valid = false;
        if (e < n_src) {
          if (bitmap != nullptr) {
            valid = raw[u] != 0;
          } else {
            id = raw[u];
            valid = (id >= 0) && (id < nb);
            bad |= !valid;
          }
        }
        const unsigned m = __ballot_sync(0xffffffffu, valid);
        if (valid) s_ids[off + __popc(m & ((1u << lane) - 1u))] = (uint16_t)id;
        off += __popc(m);
      }
    }
  }
  bad = __any_sync(0xffffffffu, bad);
  if (bad && lane == 0 && report_bad) atomicOr(status, BAS_DEV_BAD_BLOCK_ID);
  __syncwarp();
  return off;
}

__device__ __forceinline__ int warp_stage_ids(const int32_t* __restrict__ ids, const int32_t* __restrict__ count_dev,
                                              int k_host, const uint8_t* __restrict__ bitmap, int nb,
                                              uint16_t* __restrict__ s_ids, unsigned int* __restrict__ status,
                                              int lane) {
  const int none[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  return warp_stage_ids(ids, count_dev, k_host, bitmap, nb, s_ids, status, lane, false, none);
}

// System-scope 64-bit accesses to memory that another GPU of the box reads or writes through a peer
// mapping (plain per-thread loads and stores over NVLink only).  A 64-bit scalar access is single-copy
// atomic: a reader sees either the old or the new word, never a mix.
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Ranking key of a block score: unsigned keys order like the scores, with every NaN alike and
// above +infinity (torch.topk and a descending sort put NaN first), so that ranking by
// (key descending, id ascending) is a total order whatever the inputs hold.
__device__ __forceinline__ unsigned long long score_key(double s) {
  unsigned long long u = (unsigned long long)__double_as_longlong(s);
  if (s != s) u = 0x7ff8000000000000ull;
  return (u >> 63) != 0ull ? ~u : (u | 0x8000000000000000ull);
}

// fp32 -> the output's 16-bit type (round to nearest even), stored through the fp16-typed pointer
// that stands for either container.
__device__ __forceinline__ void store_out16(__half* dst, float v, bool bf16) {
  const unsigned short bits = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
  *reinterpret_cast<unsigned short*>(dst) = bits;
}

// Zero-fill of Y when the active set is empty (the reference's `out.zero_()`).
__device__ __forceinline__ void zero_output(__half* __restrict__ y, int batch, int n, long long ldy) {
  const long long total = (long long)batch * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    y[(i / n) * ldy + (i % n)] = __float2half_rn(0.f);
  }
}

}  // namespace bas
