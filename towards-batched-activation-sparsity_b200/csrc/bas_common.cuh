// Shared device helpers: mbarrier, bulk-async copies, tcgen05 wrappers and the stream-K partition
// arithmetic used by both contraction kernels.  sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bas.h"

namespace bas {

constexpr int kBlockK = BAS_BLOCK_K;                 // channels per activation block
constexpr int kTileN = BAS_TILE_N;                   // output columns per packed weight tile
constexpr int kTileBytes = kTileN * kBlockK * 2;     // one packed (block, column-tile) chunk: 16 KiB
constexpr long long kWaitCycles = 2000000000LL;      // bound of every barrier wait, about one second

// Workspace layout (bytes): [0,4) status word, [256, 256+4*kMaxTiles) arrival counters,
// [kWsHeaderBytes, ...) fp32 partial sums, two slots of [batch][128] per CTA.
constexpr int kMaxColumnTiles = 8192;                // N up to 1,048,576
constexpr size_t kWsHeaderBytes = 256 + 4 * (size_t)kMaxColumnTiles;
constexpr int kMaxGridCtas = 192;                    // persistent grid cap; partial slots are sized for it

// ---------------------------------------------------------------------------------------------
// stream-K partition: the flattened list of (column tile t, active block position i), u = t*k + i,
// is cut into G contiguous ranges of equal length (+-1); CTA c owns [part_begin(c), part_begin(c+1)).
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ long long part_begin(long long c, long long total, long long g) {
  return c * total / g;
}
// the CTA whose range contains unit u
__host__ __device__ __forceinline__ int part_owner(long long u, long long total, long long g) {
  return (int)(((u + 1) * g - 1) / total);
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

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
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

__device__ __forceinline__ int atom_add_acq_rel_gpu(int* addr, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
  return old;
}

// ---------------------------------------------------------------------------------------------
// Active-set staging: every CTA builds the same list of block ids in shared memory (16-bit).
//  * id list: copied position by position; an entry outside [0, nb) becomes kSkipId (the unit is
//    kept in the partition and contributes nothing) and is flagged in the status word;
//  * byte map: compacted in ascending order.
// All threads of the CTA must call this; returns the list length (units per column tile).
// ---------------------------------------------------------------------------------------------
constexpr uint16_t kSkipId = 0xFFFFu;

__device__ __forceinline__ int stage_active_ids(const int32_t* __restrict__ ids, const int32_t* __restrict__ count_dev,
                                                int k_host, const uint8_t* __restrict__ bitmap, int nb,
                                                uint16_t* __restrict__ s_ids, int* __restrict__ s_scan,
                                                unsigned int* __restrict__ status) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  if (bitmap == nullptr) {
    int n_src = k_host;
    if (count_dev != nullptr) n_src = min(max(__ldg(count_dev), 0), k_host);
    bool bad = false;
    for (int e = tid; e < n_src; e += blockDim.x) {
      const int id = __ldg(ids + e);
      const bool ok = (id >= 0) && (id < nb);
      s_ids[e] = ok ? (uint16_t)id : kSkipId;
      bad |= !ok;
    }
    if (bad && blockIdx.x == 0) atomicOr(status, BAS_DEV_BAD_BLOCK_ID);
    __syncthreads();
    return n_src;
  }
  // s_scan: 33 ints of scratch: [0..31] per-warp counts, [32] running base
  if (tid == 0) s_scan[32] = 0;
  __syncthreads();
  for (int base = 0; base < nb; base += blockDim.x) {
    const int e = base + tid;
    const bool valid = (e < nb) && (bitmap[e] != 0);
    const unsigned m = __ballot_sync(0xffffffffu, valid);
    if (lane == 0) s_scan[warp] = __popc(m);
    __syncthreads();
    int off = s_scan[32];
    for (int w = 0; w < warp; ++w) off += s_scan[w];
    if (valid) s_ids[off + __popc(m & ((1u << lane) - 1u))] = (uint16_t)e;
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < nwarps; ++w) tot += s_scan[w];
      s_scan[32] += tot;
    }
    __syncthreads();
  }
  return s_scan[32];
}

// Zero-fill of Y when the active set is empty (the reference's `out.zero_()`).
__device__ __forceinline__ void zero_output(__half* __restrict__ y, int batch, int n, long long ldy) {
  const long long total = (long long)batch * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    y[(i / n) * ldy + (i % n)] = __float2half_rn(0.f);
  }
}

// Rendezvous of the four warps of a 128-thread group on an mbarrier (arrival count 4), bounded.
// Orders the group's earlier memory operations before its later ones (release / acquire, CTA scope).
__device__ __forceinline__ bool group_sync(uint64_t* bar, uint32_t& phase, int lane, volatile int* abort_flag) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
  const bool ok = mbar_wait(bar, phase, abort_flag);
  phase ^= 1u;
  return ok;
}

// ---------------------------------------------------------------------------------------------
// Output of one segment (this CTA's share of column tile t) by a 128-thread group; thread r holds
// the fp32 sums v[b] of output column 128 t + r.
//  * complete segment: round and store to Y;
//  * otherwise store the fp32 partial to this CTA's slot, publish it with one release-atomic on
//    the tile's counter, and let the last contributor to arrive add all partials in CTA order and
//    store Y (so the sum never depends on arrival order).  The counter re-arms itself.
// Returns false if a bounded wait ran out.
// ---------------------------------------------------------------------------------------------
template <int NV>
__device__ __forceinline__ bool store_or_combine(float (&v)[NV], int batch, __half* __restrict__ y, long long ldy,
                                                 int n_cols, float* __restrict__ partials, int* __restrict__ counters,
                                                 int t, int t_first, bool complete, int c, int G, int k_act,
                                                 long long total, int r, int lane, uint64_t* fix_bar,
                                                 uint32_t& fix_phase, int* last_flag, volatile int* abort_flag) {
  const int col = t * kTileN + r;
  if (complete) {
    if (col < n_cols) {
#pragma unroll
      for (int b = 0; b < NV; ++b)
        if (b < batch) y[(size_t)b * ldy + col] = __float2half_rn(v[b]);
    }
    return true;
  }
  const int slot = (t == t_first) ? 0 : 1;
  float* part = partials + ((size_t)(c * 2 + slot) * batch) * kTileN;
#pragma unroll
  for (int b = 0; b < NV; ++b)
    if (b < batch) part[b * kTileN + r] = v[b];
  if (!group_sync(fix_bar, fix_phase, lane, abort_flag)) return false;
  const int cf = part_owner((long long)t * k_act, total, G);
  const int cl = part_owner((long long)(t + 1) * k_act - 1, total, G);
  if (r == 0) {
    // release: the group's partial stores (ordered before this thread by the rendezvous) become
    // visible before the count; acquire: the last arriver sees every earlier contributor's stores.
    const int old = atom_add_acq_rel_gpu(counters + t, 1);
    const int last = (old == cl - cf) ? 1 : 0;
    if (last) counters[t] = 0;   // every contributor has arrived: re-arm for the next call
    *last_flag = last;
  }
  if (!group_sync(fix_bar, fix_phase, lane, abort_flag)) return false;
  if (*last_flag) {
    constexpr int BV = NV < 8 ? NV : 8;          // batch rows per pass
    constexpr int CU = 4;                        // contributors whose loads are in flight together
#pragma unroll
    for (int b0 = 0; b0 < NV; b0 += BV) {
      if (b0 < batch) {
        float s[BV];
#pragma unroll
        for (int i = 0; i < BV; ++i) s[i] = 0.f;
        for (int cc = cf; cc <= cl; cc += CU) {
          float tmp[CU][BV];
#pragma unroll
          for (int j = 0; j < CU; ++j) {
            const int cj = min(cc + j, cl);
            const int sl = ((int)(part_begin(cj, total, G) / k_act) == t) ? 0 : 1;
            const float* pp = partials + ((size_t)(cj * 2 + sl) * batch) * kTileN + r;
#pragma unroll
            for (int i = 0; i < BV; ++i)
              tmp[j][i] = (b0 + i < batch) ? __ldcg(pp + (size_t)(b0 + i) * kTileN) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < CU; ++j) {
            if (cc + j <= cl) {                  // CTA order, independent of who arrived when
#pragma unroll
              for (int i = 0; i < BV; ++i) s[i] += tmp[j][i];
            }
          }
        }
        if (col < n_cols) {
#pragma unroll
          for (int i = 0; i < BV; ++i)
            if (b0 + i < batch) y[(size_t)(b0 + i) * ldy + col] = __float2half_rn(s[i]);
        }
      }
    }
  }
  return true;
}

}  // namespace bas
