// Split-K GEMV-style kernel for decode batches of 1..8 rows (CUDA cores, fp32 accumulate).
//
// Persistent grid of one CTA per SM.  The flattened (column tile, active block) list is cut into
// equal contiguous ranges (stream-K); each CTA streams its 16 KiB weight tiles with bulk-async
// copies through an mbarrier ring and keeps one fp32 accumulator per (row of the tile, batch row).
// A column tile whose blocks are spread over several CTAs is combined without atomics: every
// contributor stores an fp32 partial, the last one to arrive (per-tile counter) adds all partials
// in CTA order and writes fp16, so the result does not depend on arrival order.
//
// Roles: warp 0 issues the copies, warp 1 widens each tile's activation slice to fp32, warps 2..9
// are two consumer groups that take alternate tiles.  Every wait is on an mbarrier and bounded; no
// bar.sync is used once the roles have split, so a lost arrival ends in an error flag, not a hang.
//
// Replaces, for small batches, the reference's index-list kernel and its split-K write + reduce
// pair (kernels/shared_mask_batched_triton_min_runtime.py:684-733, 1898-1988).
#include "bas_kernels.cuh"

namespace bas {

namespace {

constexpr int kGroupThreads = 128;
constexpr int kGemvThreads = 64 + 2 * kGroupThreads;

template <int B>
struct GemvCfg {
  static constexpr int kXBytes = B * 128;                 // one 64-channel fp16 slice per batch row
  static constexpr int kXfBytes = B * 256;                // the same slice widened to fp32
  static constexpr int kStageBytes = kTileBytes + kXBytes + kXfBytes;
  static constexpr int kStagesRaw = (184 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
  static constexpr int kExchFloats = 2 * B * 128;         // [segment parity][B][128] fp32
};

struct GemvSmemHeader {
  uint64_t full[16];      // weights + fp16 activations have landed (bytes)
  uint64_t xready[16];    // fp32 activations written by the converter warp
  uint64_t empty[16];     // the consuming group is done with the stage
  uint64_t exch_full[2];  // group 1 has published its segment sums
  uint64_t exch_empty[2]; // group 0 has read them
  uint64_t fix_bar;       // group-0 rendezvous of the split-K combine
  int scan[34];
  int abort_flag;
  int last_flag;
};

__host__ __device__ inline size_t gemv_ids_bytes(int nb) { return ((size_t)nb * 2 + 127) / 128 * 128; }

template <int B>
size_t gemv_smem_bytes(int nb) {
  return 128 /*alignment slack*/ + (sizeof(GemvSmemHeader) + 127) / 128 * 128 + gemv_ids_bytes(nb) +
         sizeof(float) * GemvCfg<B>::kExchFloats + (size_t)GemvCfg<B>::kStages * GemvCfg<B>::kStageBytes;
}

template <int B>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_splitk_kernel(const GemmParams p) {
  using Cfg = GemvCfg<B>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sp = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  GemvSmemHeader* hdr = (GemvSmemHeader*)sp;
  sp += (sizeof(GemvSmemHeader) + 127) / 128 * 128;
  uint16_t* s_ids = (uint16_t*)sp;
  sp += gemv_ids_bytes(p.nb);
  float* s_exch = (float*)sp;
  sp += sizeof(float) * Cfg::kExchFloats;
  uint8_t* s_stage = sp;  // 128-byte aligned; per stage: [16 KiB weights][B*128 fp16 x][B*256 fp32 x]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &hdr->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->xready[s], 1);
      mbar_init(&hdr->empty[s], kGroupThreads / 32);
    }
    for (int e = 0; e < 2; ++e) {
      mbar_init(&hdr->exch_full[e], kGroupThreads / 32);
      mbar_init(&hdr->exch_empty[e], kGroupThreads / 32);
    }
    mbar_init(&hdr->fix_bar, kGroupThreads / 32);
    hdr->abort_flag = 0;
    hdr->last_flag = 0;
    fence_barrier_init();
  }
  // Nothing above touches global memory.  The id list may be the previous kernel's output unless
  // the caller declared it stable; X, the workspace and Y always wait.
  const bool early_ids = (p.flags & kFlagStableIds) != 0 && p.count_dev == nullptr;
  if (!early_ids) pdl_wait();
  const int k_act = stage_active_ids(p.ids, p.count_dev, p.k_host, p.bitmap, p.nb, s_ids, hdr->scan, p.status);
  pdl_launch_dependents();

  if (k_act == 0) {
    if (early_ids) pdl_wait();
    zero_output(p.y, p.batch, p.n, p.ldy);
    return;
  }
  const long long total = (long long)k_act * p.nt;
  // Never more ranges than units: every participating CTA then owns at least one unit, so the
  // contributors of a column tile are a contiguous run of CTAs.
  const int c = blockIdx.x, G = (int)min((long long)gridDim.x, total);
  if (c >= G) return;
  const long long u0 = part_begin(c, total, G), u1 = part_begin(c + 1, total, G);
  const int cnt = (int)(u1 - u0);

  int issued = 0;   // tiles whose copies the producer thread has started
  if (warp == 0) {
    // ------------------------------ producer (one thread) ------------------------------
    if (lane == 0) {
      int m = 0, n0 = 0;
      if (early_ids) {
        // The ids are not the previous kernel's output: stream the first ring-full of weight tiles
        // while that kernel is still draining, then wait for it before touching the activations.
        int ahead = 0;
        for (int n = 0; n < cnt && ahead < S; ++n) {
          const long long u = u0 + n;
          const int t = (int)(u / k_act), j = s_ids[(int)(u - (long long)t * k_act)];
          if (j == kSkipId) continue;
          const int kvalid = min(kBlockK, p.k - j * kBlockK);
          mbar_arrive_expect_tx(&hdr->full[ahead], kTileBytes + B * kvalid * 2);
          bulk_copy_g2s(s_stage + (size_t)ahead * Cfg::kStageBytes, p.packed + ((size_t)j * p.nt + t) * kTileBytes,
                        kTileBytes, &hdr->full[ahead]);
          ++ahead;
        }
        issued = ahead;
        pdl_wait();
        for (; n0 < cnt && m < ahead; ++n0) {
          const long long u = u0 + n0;
          const int j = s_ids[(int)(u % k_act)];
          if (j == kSkipId) continue;
          const int kvalid = min(kBlockK, p.k - j * kBlockK);
          uint8_t* st = s_stage + (size_t)m * Cfg::kStageBytes;
#pragma unroll
          for (int b = 0; b < B; ++b) {
            bulk_copy_g2s(st + kTileBytes + b * 128, p.x + (size_t)b * p.ldx + (size_t)j * kBlockK, kvalid * 2,
                          &hdr->full[m]);
          }
          ++m;
        }
      }
      for (int n = n0; n < cnt; ++n) {
        const long long u = u0 + n;
        const int t = (int)(u / k_act), i = (int)(u - (long long)t * k_act);
        const int j = s_ids[i];
        if (j == kSkipId) continue;
        const int s = m % S;
        if (m >= S && !mbar_wait(&hdr->empty[s], ((m / S) - 1) & 1, abort_flag)) {
          atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
          hdr->abort_flag = 1;
          break;
        }
        const int kvalid = min(kBlockK, p.k - j * kBlockK);
        uint8_t* st = s_stage + (size_t)s * Cfg::kStageBytes;
        mbar_arrive_expect_tx(&hdr->full[s], kTileBytes + B * kvalid * 2);
        bulk_copy_g2s(st, p.packed + ((size_t)j * p.nt + t) * kTileBytes, kTileBytes, &hdr->full[s]);
#pragma unroll
        for (int b = 0; b < B; ++b) {
          bulk_copy_g2s(st + kTileBytes + b * 128, p.x + (size_t)b * p.ldx + (size_t)j * kBlockK, kvalid * 2,
                        &hdr->full[s]);
        }
        issued = ++m;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ converter: fp16 -> fp32 activations ------------------------------
    int m = 0;
    for (int n = 0; n < cnt; ++n) {
      const long long u = u0 + n;
      const int j = s_ids[(int)(u % k_act)];
      if (j == kSkipId) continue;
      const int s = m % S;
      if (!mbar_wait(&hdr->full[s], (m / S) & 1, abort_flag)) {
        atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
        hdr->abort_flag = 1;
        break;
      }
      const int kvalid = min(kBlockK, p.k - j * kBlockK);
      const uint8_t* st = s_stage + (size_t)s * Cfg::kStageBytes;
      float* xf = (float*)(st + kTileBytes + Cfg::kXBytes);
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const __half2 h = *(const __half2*)(st + kTileBytes + b * 128 + lane * 4);
        float2 f = __half22float2(h);
        if (2 * lane >= kvalid) f = make_float2(0.f, 0.f);  // channels past K of a ragged last block
        *(float2*)(xf + b * 64 + 2 * lane) = f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&hdr->xready[s]);
      ++m;
    }
  } else {
    // ------------------------------ consumers ------------------------------
    const int ct = tid - 64;
    const int g = ct >> 7;     // group 0 / 1 takes the even / odd tiles of this CTA's range
    const int r = ct & 127;    // row of the weight tile = output column within the tile
    float acc[B][2];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b][0] = acc[b][1] = 0.f;
    int seg = 0, m = 0;
    int seg_i0 = (int)(u0 % k_act);
    const int t_first = (int)(u0 / k_act);
    uint32_t fix_phase = 0;
    bool ok = true;
    if (early_ids) pdl_wait();   // before the first write to the workspace or Y

    for (int n = 0; n < cnt && ok; ++n) {
      const long long u = u0 + n;
      const int t = (int)(u / k_act), i = (int)(u - (long long)t * k_act);
      const bool skip = s_ids[i] == kSkipId;
      if (!skip && (m & 1) == g) {
        const int s = m % S;
        // xready implies full (the converter waited on it); observing full directly as well makes
        // the bulk copy's writes visible to this thread without relying on transitivity.
        if (!mbar_wait(&hdr->xready[s], (m / S) & 1, abort_flag) ||
            !mbar_wait(&hdr->full[s], (m / S) & 1, abort_flag)) {
          ok = false;
          break;
        }
        const uint8_t* st = s_stage + (size_t)s * Cfg::kStageBytes;
        const float* xf = (const float*)(st + kTileBytes + Cfg::kXBytes);
        const uint8_t* wrow = st + r * 128;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint4 v = *(const uint4*)(wrow + ((q ^ (r & 7)) << 4));
          const float2 w01 = __half22float2(*(const __half2*)&v.x);
          const float2 w23 = __half22float2(*(const __half2*)&v.y);
          const float2 w45 = __half22float2(*(const __half2*)&v.z);
          const float2 w67 = __half22float2(*(const __half2*)&v.w);
#pragma unroll
          for (int b = 0; b < B; ++b) {
            const float4 xa = *(const float4*)(xf + b * 64 + q * 8);
            const float4 xb = *(const float4*)(xf + b * 64 + q * 8 + 4);
            acc[b][0] = fmaf(w01.x, xa.x, acc[b][0]);
            acc[b][1] = fmaf(w01.y, xa.y, acc[b][1]);
            acc[b][0] = fmaf(w23.x, xa.z, acc[b][0]);
            acc[b][1] = fmaf(w23.y, xa.w, acc[b][1]);
            acc[b][0] = fmaf(w45.x, xb.x, acc[b][0]);
            acc[b][1] = fmaf(w45.y, xb.y, acc[b][1]);
            acc[b][0] = fmaf(w67.x, xb.z, acc[b][0]);
            acc[b][1] = fmaf(w67.y, xb.w, acc[b][1]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->empty[s]);
      }
      if (!skip) ++m;

      if (i == k_act - 1 || n == cnt - 1) {
        // ---- end of a segment: all of this CTA's blocks of column tile t ----
        float v[B];
#pragma unroll
        for (int b = 0; b < B; ++b) v[b] = acc[b][0] + acc[b][1];
        const int e = seg & 1;
        float* ex = s_exch + e * B * 128;
        if (g == 1) {
          if (seg >= 2 && !mbar_wait(&hdr->exch_empty[e], ((seg >> 1) - 1) & 1, abort_flag)) {
            ok = false;
            break;
          }
#pragma unroll
          for (int b = 0; b < B; ++b) ex[b * 128 + r] = v[b];
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->exch_full[e]);
        } else {
          if (!mbar_wait(&hdr->exch_full[e], (seg >> 1) & 1, abort_flag)) {
            ok = false;
            break;
          }
#pragma unroll
          for (int b = 0; b < B; ++b) v[b] += ex[b * 128 + r];   // fixed order: group 0 + group 1
          __syncwarp();
          if (lane == 0) mbar_arrive(&hdr->exch_empty[e]);
          const bool complete = (seg_i0 == 0) && (i == k_act - 1);
          if (!store_or_combine<B>(v, B, p.y, p.ldy, p.n, p.partials, p.counters, t, t_first, complete, c, G, k_act,
                                   total, r, lane, &hdr->fix_bar, fix_phase, &hdr->last_flag, abort_flag)) {
            ok = false;
            break;
          }
        }
#pragma unroll
        for (int b = 0; b < B; ++b) acc[b][0] = acc[b][1] = 0.f;
        ++seg;
        seg_i0 = 0;
      }
    }
    if (!ok) {
      atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
      hdr->abort_flag = 1;
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
cudaError_t launch_gemv_b(const GemmParams& p, int sm_count, cudaStream_t stream) {
  const size_t smem = gemv_smem_bytes<B>(p.nb);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(gemv_splitk_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  const long long units = (long long)(p.bitmap != nullptr ? p.nb : p.k_host) * p.nt;
  const int grid = (int)(units < sm_count ? (units < 1 ? 1 : units) : sm_count);
  count_launch();
  return launch_with_pdl(gemv_splitk_kernel<B>, grid, kGemvThreads, smem, stream, p);
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
