// CUDA-core kernel for decode batches of 1..8 rows (fp32 accumulate).
//
// Work split: the output columns are cut into one contiguous range per CTA (about N / #SMs columns);
// a CTA walks ALL active blocks for its range and keeps the fp32 sums in registers, so no CTA needs
// another's partial sums: no workspace, no atomics, and the result cannot depend on timing.
// For block j the CTA's weights are rows n0..n1 of the packed layout: one contiguous chunk of
// (n1 - n0) x 128 bytes fetched by a single bulk-async copy; the batch's 64-channel activation
// slices ride on the same mbarrier.  With chunks of ~4 KiB the ring holds up to 32 of them, i.e.
// most of a CTA's share is in flight at once.
//
// Roles: warp 0 stages the id list and issues the copies, warp 1 widens each block's activation
// slice to fp32 once per CTA, warps 2..9 compute: thread (r, q) owns 16-byte chunk q of weight row
// r (8 channels) and all batch rows; the 8 threads of a row are adjacent lanes and add their sums
// with shuffles at the end.  Every wait is a bounded mbarrier wait.
//
// Replaces, for small batches, the reference's index-list kernel and its split-K write + reduce
// pair (kernels/shared_mask_batched_triton_min_runtime.py:684-733, 1898-1988).
#include "bas_kernels.cuh"

namespace bas {

namespace {

constexpr int kConsumerThreads = 256;
constexpr int kGemvThreads = 64 + kConsumerThreads;
constexpr int kMaxPairs = (kTileN * 8) / kConsumerThreads;   // (row, chunk) pairs per thread for a 128-wide sub-tile
constexpr size_t kSmemBudget = 224 * 1024;

struct GemvSmemHeader {
  uint64_t full[kMaxStages];      // weights + fp16 activations have landed (bytes)
  uint64_t xready[kMaxStages];    // fp32 activations written by the converter warp
  uint64_t empty[kMaxStages];     // all consumer warps are done with the slot
  uint64_t ids_ready;
  int k_act;
  int abort_flag;
};

inline size_t gemv_fixed_smem(int nb) {
  return 128 /*alignment slack*/ + (sizeof(GemvSmemHeader) + 127) / 128 * 128 + ((size_t)nb * 2 + 127) / 128 * 128;
}

template <int B>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_colsplit_kernel(const GemmParams p) {
  constexpr int kXBytes = B * 128;    // fp16 slices
  constexpr int kXfBytes = B * 256;   // fp32 slices
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sp = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  GemvSmemHeader* hdr = (GemvSmemHeader*)sp;
  sp += (sizeof(GemvSmemHeader) + 127) / 128 * 128;
  uint16_t* s_ids = (uint16_t*)sp;
  sp += ((size_t)p.nb * 2 + 127) / 128 * 128;
  uint8_t* s_stage = sp;   // 128-byte aligned; a slot holds `group` tiles of [wslot weights][B*128 fp16 x][B*256 fp32 x]
  const int S = p.stages, G = p.group;
  const int tile_bytes = p.wslot + kXBytes + kXfBytes;
  const int stage_bytes = G * tile_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &hdr->abort_flag;

  if (tid < S) {
    mbar_init(&hdr->full[tid], 1);
    mbar_init(&hdr->xready[tid], 1);
    mbar_init(&hdr->empty[tid], kConsumerThreads / 32);
    fence_barrier_init();
  } else if (tid == 64) {
    mbar_init(&hdr->ids_ready, 1);
    hdr->abort_flag = 0;
    hdr->k_act = 0;
    fence_barrier_init();
  }
  __syncthreads();

  const int units = p.npad >> 3;
  const int n0 = col_begin(blockIdx.x, units, p.ranges), n1 = col_begin(blockIdx.x + 1, units, p.ranges);
  const int width = n1 - n0;
  const int n_sub = (width + kTileN - 1) / kTileN;

  // Nothing so far touched global memory.  The id list may be the previous kernel's output unless
  // the caller declared it stable; X and Y always wait for the previous kernel.
  const bool early_ids = (p.flags & kFlagStableIds) != 0 && p.count_dev == nullptr;
  int armed = 0;   // ring slots (groups) whose copies the producer thread has started

  if (warp == 0) {
    // ------------------------------ id staging + producer ------------------------------
    if (!early_ids) pdl_wait();
    const int k_act = warp_stage_ids(p.ids, p.count_dev, p.k_host, p.bitmap, p.nb, s_ids, p.status, lane);
    if (lane == 0) {
      hdr->k_act = k_act;
      mbar_arrive(&hdr->ids_ready);
    }
    pdl_launch_dependents();
    const int M = n_sub * k_act;                 // tiles of this CTA: sub-tile major, active block minor
    const int NG = (M + G - 1) / G;              // groups = barrier hand-offs
    if (M > 0) {
      // One pass per ring slot.  Lane l owns tile l of the slot's group: it works out that tile's
      // addresses (the integer divisions run side by side in the lanes), the byte counts are added
      // across the warp, lane 0 waits for the slot and arms its barrier, then every lane issues its
      // tile's weight chunk and activation slices.  Slot index and phase are carried along.
      int s = 0, ph = 0;   // slot of group g and the parity of its previous use
      auto lane_tile = [&](int g, int& sub, int& j, int& wbytes, int& xbytes) -> bool {
        const int m = g * G + lane;
        if (lane >= G || m >= M) return false;
        sub = (n_sub == 1) ? 0 : m / k_act;
        j = s_ids[m - sub * k_act];
        wbytes = min(kTileN, width - sub * kTileN) * kRowBytes;
        xbytes = min(kBlockK, p.k - j * kBlockK) * 2;
        return true;
      };
      auto issue_x = [&](uint8_t* st, int j, int xbytes, uint64_t* bar) {
#pragma unroll
        for (int b = 0; b < B; ++b)
          bulk_copy_g2s(st + p.wslot + b * 128, p.x + (size_t)b * p.ldx + (size_t)j * kBlockK, xbytes, bar);
      };
      int g0 = 0;
      if (early_ids) {
        // Stream the first ring-full of weight chunks while the previous kernel is still draining,
        // then wait for it before touching the activations.
        const int ahead = min(S, NG);
        for (int g = 0; g < ahead; ++g) {
          int sub = 0, j = 0, wbytes = 0, xbytes = 0;
          const bool have = lane_tile(g, sub, j, wbytes, xbytes);
          const int total = __reduce_add_sync(0xffffffffu, have ? wbytes + B * xbytes : 0);
          if (lane == 0) mbar_arrive_expect_tx(&hdr->full[g], total);
          __syncwarp();
          if (have)
            bulk_copy_g2s(s_stage + (size_t)g * stage_bytes + (size_t)lane * tile_bytes,
                          p.packed + ((size_t)j * p.npad + n0 + sub * kTileN) * kRowBytes, wbytes, &hdr->full[g]);
        }
        armed = ahead;
        pdl_wait();
        for (int g = 0; g < ahead; ++g) {
          int sub = 0, j = 0, wbytes = 0, xbytes = 0;
          if (lane_tile(g, sub, j, wbytes, xbytes))
            issue_x(s_stage + (size_t)g * stage_bytes + (size_t)lane * tile_bytes, j, xbytes, &hdr->full[g]);
        }
        g0 = ahead;
        s = (ahead == S) ? 0 : ahead;
      }
      for (int g = g0; g < NG; ++g) {
        int sub = 0, j = 0, wbytes = 0, xbytes = 0;
        const bool have = lane_tile(g, sub, j, wbytes, xbytes);
        const int total = __reduce_add_sync(0xffffffffu, have ? wbytes + B * xbytes : 0);
        bool ok = true;
        if (lane == 0) {
          if (g >= S) ok = mbar_wait_for(&hdr->empty[s], ph, abort_flag, p.wait_cycles);
          if (ok) mbar_arrive_expect_tx(&hdr->full[s], total);
        }
        if (!__shfl_sync(0xffffffffu, ok, 0)) {
          if (lane == 0) {
            atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
            hdr->abort_flag = 1;
          }
          break;
        }
        if (have) {
          uint8_t* st = s_stage + (size_t)s * stage_bytes + (size_t)lane * tile_bytes;
          bulk_copy_g2s(st, p.packed + ((size_t)j * p.npad + n0 + sub * kTileN) * kRowBytes, wbytes, &hdr->full[s]);
          issue_x(st, j, xbytes, &hdr->full[s]);
        }
        armed = g + 1;
        if (++s == S) {   // next slot; from the second lap on its previous use must have been released
          s = 0;
          if (g >= S) ph ^= 1;
        }
      }
    }
  } else {
    bool ok = __all_sync(0xffffffffu, mbar_wait_for(&hdr->ids_ready, 0, abort_flag, p.wait_cycles));
    const int k_act = ok ? hdr->k_act : 0;
    const int M = n_sub * k_act;
    const int NG = (M + G - 1) / G;

    if (warp == 1) {
      // ------------------------------ converter: fp16 -> fp32 activations ------------------------------
      int s = 0, fph = 0;
      for (int g = 0; g < NG && ok; ++g) {
        // the verdict is made warp-uniform so that the warp-level primitives below stay converged
        if (!__all_sync(0xffffffffu, mbar_wait_for(&hdr->full[s], fph, abort_flag, p.wait_cycles))) {
          ok = false;
          break;
        }
        const int cnt = min(M, (g + 1) * G) - g * G;
        for (int t = 0; t < cnt; ++t) {
          int mm = g * G + t;
          if (n_sub > 1) mm %= k_act;
          const int j = s_ids[mm];
          const int kvalid = min(kBlockK, p.k - j * kBlockK);
          const uint8_t* xh = s_stage + (size_t)s * stage_bytes + (size_t)t * tile_bytes + p.wslot;
          float* xf = (float*)(xh + kXBytes);
#pragma unroll
          for (int b = 0; b < B; ++b) {
            float2 f = __half22float2(*(const __half2*)(xh + b * 128 + lane * 4));
            if (2 * lane >= kvalid) f = make_float2(0.f, 0.f);   // channels past K of a ragged last block
            *(float2*)(xf + b * 64 + 2 * lane) = f;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->xready[s]);
        if (++s == S) {
          s = 0;
          fph ^= 1;
        }
      }
      if (!ok) {
        atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
        hdr->abort_flag = 1;
      }
    } else {
      // ------------------------------ consumers ------------------------------
      const int ct = tid - 64;
      if (early_ids) pdl_wait();   // before the first write to Y
      if (ok && k_act == 0) {
        const long long total = (long long)p.batch * p.n;
        for (long long e = (long long)blockIdx.x * kConsumerThreads + ct; e < total;
             e += (long long)gridDim.x * kConsumerThreads)
          p.y[(e / p.n) * p.ldy + (e % p.n)] = __float2half_rn(0.f);
      }
      int m = 0, s = 0, pos = 0, fph = 0;   // tile, its slot, position in the slot's group, slot parity
      for (int sub = 0; sub < n_sub && ok && k_act > 0; ++sub) {
        const int wsub = min(kTileN, width - sub * kTileN);
        const int npairs = wsub * 8;                 // (row, 16-byte chunk) pairs of this sub-tile
        float acc[kMaxPairs][B];
#pragma unroll
        for (int e = 0; e < kMaxPairs; ++e)
#pragma unroll
          for (int b = 0; b < B; ++b) acc[e][b] = 0.f;

        for (int i = 0; i < k_act; ++i, ++m) {
          if (pos == 0 || i == 0) {
            // xready is arrived by the converter after it has seen the slot's copies land; a slot that
            // straddles two sub-tiles is waited for again, which returns at once.
            if (!__all_sync(0xffffffffu, mbar_wait_for(&hdr->xready[s], fph, abort_flag, p.wait_cycles) &&
                                             mbar_wait_for(&hdr->full[s], fph, abort_flag, p.wait_cycles))) {
              ok = false;
              break;
            }
          }
          const uint8_t* st = s_stage + (size_t)s * stage_bytes + (size_t)pos * tile_bytes;
          const float* xf = (const float*)(st + p.wslot + kXBytes);
#pragma unroll
          for (int e = 0; e < kMaxPairs; ++e) {
            const int pr = ct + e * kConsumerThreads;
            if (pr < npairs) {
              const int r = pr >> 3, q = pr & 7;
              const uint4 v = *(const uint4*)(st + r * kRowBytes + ((q ^ (r & 7)) << 4));
              const float2 w01 = __half22float2(*(const __half2*)&v.x);
              const float2 w23 = __half22float2(*(const __half2*)&v.y);
              const float2 w45 = __half22float2(*(const __half2*)&v.z);
              const float2 w67 = __half22float2(*(const __half2*)&v.w);
#pragma unroll
              for (int b = 0; b < B; ++b) {
                const float4 xa = *(const float4*)(xf + b * 64 + q * 8);
                const float4 xb = *(const float4*)(xf + b * 64 + q * 8 + 4);
                float a0 = acc[e][b];
                a0 = fmaf(w01.x, xa.x, a0);
                a0 = fmaf(w01.y, xa.y, a0);
                a0 = fmaf(w23.x, xa.z, a0);
                a0 = fmaf(w23.y, xa.w, a0);
                a0 = fmaf(w45.x, xb.x, a0);
                a0 = fmaf(w45.y, xb.y, a0);
                a0 = fmaf(w67.x, xb.z, a0);
                a0 = fmaf(w67.y, xb.w, a0);
                acc[e][b] = a0;
              }
            }
          }
          if (pos == G - 1 || m == M - 1) {   // last tile of the slot: hand it back
            __syncwarp();
            if (lane == 0) mbar_arrive(&hdr->empty[s]);
            pos = 0;
            if (++s == S) {
              s = 0;
              fph ^= 1;
            }
          } else {
            ++pos;
          }
        }
        if (!ok) break;
        // the 8 chunk-threads of a row are lanes 8g .. 8g+7: add their sums, lane 8g stores
#pragma unroll
        for (int e = 0; e < kMaxPairs; ++e) {
          const int pr = ct + e * kConsumerThreads;
          const int r = pr >> 3;
          const int col = n0 + sub * kTileN + r;
#pragma unroll
          for (int b = 0; b < B; ++b) {
            float v = acc[e][b];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            if ((pr & 7) == 0 && pr < npairs && col < p.n) p.y[(size_t)b * p.ldy + col] = __float2half_rn(v);
          }
        }
      }
      if (!ok) {
        atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
        hdr->abort_flag = 1;
      }
    }
  }

  __syncwarp();   // warps with single-lane roles join the barrier whole
  __syncthreads();
  if (hdr->abort_flag != 0 && tid == 0) {
    // Gave up somewhere: do not leave while bulk copies may still be landing in this CTA's memory.
    int zero = 0;
    for (int g = max(0, armed - S); g < armed; ++g) (void)mbar_wait_for(&hdr->full[g % S], (g / S) & 1, &zero, p.wait_cycles);
  }
}

template <int B>
cudaError_t launch_gemv_b(GemmParams p, int sm_count, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(gemv_colsplit_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  const int units = p.npad / 8;
  p.cluster = 1;
  p.ranges = sm_count < units ? sm_count : units;
  const int wmax = ((units + p.ranges - 1) / p.ranges) * 8;
  const int wsub_max = wmax < kTileN ? wmax : kTileN;
  p.wslot = (wsub_max * kRowBytes + 127) / 128 * 128;
  const size_t fixed = gemv_fixed_smem(p.nb);
  const size_t stage_bytes = (size_t)p.wslot + B * 128 + B * 256;
  if (fixed + 2 * stage_bytes > kSmemBudget) return cudaErrorInvalidValue;
  // One barrier hand-off costs a few hundred cycles per role: a slot gathers enough blocks (about
  // 24 KiB) for the hand-offs to stay off the critical path.
  int group = (int)((24 * 1024 + stage_bytes - 1) / stage_bytes);
  if (group > 16) group = 16;
  if (group < 1) group = 1;
  int stages = (int)((kSmemBudget - fixed) / (stage_bytes * group));
  if (stages < 2) {
    group = 1;
    stages = (int)((kSmemBudget - fixed) / stage_bytes);
  }
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  p.group = group;
  const size_t smem = fixed + (size_t)stages * group * stage_bytes;
  count_launch();
  return launch_with_pdl(gemv_colsplit_kernel<B>, p.ranges, kGemvThreads, smem, 1, stream, p);
}

}  // namespace

cudaError_t launch_gemv(const GemmParams& p, int sm_count, cudaStream_t stream) {
  switch (p.batch) {
    case 1: return launch_gemv_b<1>(p, sm_count, stream);
    case 2: return launch_gemv_b<2>(p, sm_count, stream);
    case 3: return launch_gemv_b<3>(p, sm_count, stream);
    case 4: return launch_gemv_b<4>(p, sm_count, stream);
    case 5: return launch_gemv_b<5>(p, sm_count, stream);
    case 6: return launch_gemv_b<6>(p, sm_count, stream);
    case 7: return launch_gemv_b<7>(p, sm_count, stream);
    case 8: return launch_gemv_b<8>(p, sm_count, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace bas
