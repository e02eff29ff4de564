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
  uint8_t* s_stage = sp;   // 128-byte aligned; per slot: [wslot weights][B*128 fp16 x][B*256 fp32 x]
  const int S = p.stages;
  const int stage_bytes = p.wslot + kXBytes + kXfBytes;

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
  int issued = 0;   // slots whose copies the producer thread has started

  if (warp == 0) {
    // ------------------------------ id staging + producer ------------------------------
    if (!early_ids) pdl_wait();
    const int k_act = warp_stage_ids(p.ids, p.count_dev, p.k_host, p.bitmap, p.nb, s_ids, p.status, lane);
    if (lane == 0) {
      hdr->k_act = k_act;
      mbar_arrive(&hdr->ids_ready);
    }
    pdl_launch_dependents();
    const int cnt = n_sub * k_act;
    if (lane == 0 && cnt > 0) {
      int m = 0, n_resume = 0;
      if (early_ids) {
        // Stream the first ring-full of weight chunks while the previous kernel is still draining,
        // then wait for it before touching the activations.
        int ahead = 0;
        for (int n = 0; n < cnt && ahead < S; ++n) {
          const int sub = n / k_act, j = s_ids[n - sub * k_act];
          if (j == kSkipId) continue;
          const int wsub = min(kTileN, width - sub * kTileN);
          const int kvalid = min(kBlockK, p.k - j * kBlockK);
          mbar_arrive_expect_tx(&hdr->full[ahead], wsub * kRowBytes + B * kvalid * 2);
          bulk_copy_g2s(s_stage + (size_t)ahead * stage_bytes,
                        p.packed + ((size_t)j * p.npad + n0 + sub * kTileN) * kRowBytes, wsub * kRowBytes,
                        &hdr->full[ahead]);
          ++ahead;
        }
        issued = ahead;
        pdl_wait();
        for (; n_resume < cnt && m < ahead; ++n_resume) {
          const int j = s_ids[n_resume % k_act];
          if (j == kSkipId) continue;
          const int kvalid = min(kBlockK, p.k - j * kBlockK);
          uint8_t* st = s_stage + (size_t)m * stage_bytes + p.wslot;
#pragma unroll
          for (int b = 0; b < B; ++b)
            bulk_copy_g2s(st + b * 128, p.x + (size_t)b * p.ldx + (size_t)j * kBlockK, kvalid * 2, &hdr->full[m]);
          ++m;
        }
      }
      for (int n = n_resume; n < cnt; ++n) {
        const int sub = n / k_act, j = s_ids[n - sub * k_act];
        if (j == kSkipId) continue;
        const int s = m % S;
        if (m >= S && !mbar_wait(&hdr->empty[s], ((m / S) - 1) & 1, abort_flag)) {
          atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
          hdr->abort_flag = 1;
          break;
        }
        const int wsub = min(kTileN, width - sub * kTileN);
        const int kvalid = min(kBlockK, p.k - j * kBlockK);
        uint8_t* st = s_stage + (size_t)s * stage_bytes;
        mbar_arrive_expect_tx(&hdr->full[s], wsub * kRowBytes + B * kvalid * 2);
        bulk_copy_g2s(st, p.packed + ((size_t)j * p.npad + n0 + sub * kTileN) * kRowBytes, wsub * kRowBytes,
                      &hdr->full[s]);
#pragma unroll
        for (int b = 0; b < B; ++b)
          bulk_copy_g2s(st + p.wslot + b * 128, p.x + (size_t)b * p.ldx + (size_t)j * kBlockK, kvalid * 2,
                        &hdr->full[s]);
        issued = ++m;
      }
    }
  } else {
    bool ok = __all_sync(0xffffffffu, mbar_wait(&hdr->ids_ready, 0, abort_flag));
    const int k_act = ok ? hdr->k_act : 0;

    if (warp == 1) {
      // ------------------------------ converter: fp16 -> fp32 activations ------------------------------
      int m = 0;
      for (int n = 0; n < n_sub * k_act && ok; ++n) {
        const int j = s_ids[n % k_act];
        if (j == kSkipId) continue;
        const int s = m % S;
        // the verdict is made warp-uniform so that the warp-level primitives below stay converged
        if (!__all_sync(0xffffffffu, mbar_wait(&hdr->full[s], (m / S) & 1, abort_flag))) {
          ok = false;
          break;
        }
        const int kvalid = min(kBlockK, p.k - j * kBlockK);
        const uint8_t* xh = s_stage + (size_t)s * stage_bytes + p.wslot;
        float* xf = (float*)(xh + kXBytes);
#pragma unroll
        for (int b = 0; b < B; ++b) {
          float2 f = __half22float2(*(const __half2*)(xh + b * 128 + lane * 4));
          if (2 * lane >= kvalid) f = make_float2(0.f, 0.f);   // channels past K of a ragged last block
          *(float2*)(xf + b * 64 + 2 * lane) = f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->xready[s]);
        ++m;
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
      int m = 0;
      for (int sub = 0; sub < n_sub && ok && k_act > 0; ++sub) {
        const int wsub = min(kTileN, width - sub * kTileN);
        const int npairs = wsub * 8;                 // (row, 16-byte chunk) pairs of this sub-tile
        float acc[kMaxPairs][B];
#pragma unroll
        for (int e = 0; e < kMaxPairs; ++e)
#pragma unroll
          for (int b = 0; b < B; ++b) acc[e][b] = 0.f;

        for (int i = 0; i < k_act; ++i) {
          if (s_ids[i] == kSkipId) continue;
          const int s = m % S;
          // xready implies full (the converter waited on it); observing full directly as well makes
          // the bulk copy's writes visible to this thread without relying on transitivity.
          // (The verdict is made warp-uniform so that the warp-level primitives stay converged.)
          const bool landed = mbar_wait(&hdr->xready[s], (m / S) & 1, abort_flag) &&
                              mbar_wait(&hdr->full[s], (m / S) & 1, abort_flag);
          if (!__all_sync(0xffffffffu, landed)) {
            ok = false;
            break;
          }
          const uint8_t* st = s_stage + (size_t)s * stage_bytes;
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
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->empty[s]);
          ++m;
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

  __syncthreads();
  if (hdr->abort_flag != 0 && tid == 0) {
    // Gave up somewhere: do not leave while bulk copies may still be landing in this CTA's memory.
    int zero = 0;
    for (int n = max(0, issued - S); n < issued; ++n) (void)mbar_wait(&hdr->full[n % S], (n / S) & 1, &zero);
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
  int stages = (int)((kSmemBudget - fixed) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  const size_t smem = fixed + (size_t)stages * stage_bytes;
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
