// Swapped-operand tcgen05 kernel for decode batches of 9..64 rows.
//
// The 128 output columns of a packed weight tile are the MMA's M dimension, the (padded) batch is
// its N dimension, and each 64-channel block is four K=16 steps:
//     D[128 x Bpad] (TMEM, fp32) += Wtile[128 x 64] (smem, K-major, 128B swizzle) * Xtile[Bpad x 64]^T
// Weight tiles arrive by 1-D bulk copies of 16 KiB (they are stored pre-swizzled), activation tiles
// by a 2-D tensor-map copy straight from X[batch, K] with the same swizzle; rows past the batch and
// channels past K arrive as zeros.  Work split, stream-K ranges and the order-independent split-K
// combine are the same as in the small-batch kernel.
//
// Roles: warp 0 issues copies, warp 1 issues MMAs (one elected thread each), warps 2..5 drain the
// accumulators (tcgen05.ld), two accumulator buffers let a drain overlap the next segment's MMAs.
// All waits are bounded mbarrier waits; TMEM is released on every path.
//
// Replaces, for larger batches, the reference's bitmap/index-list tl.dot kernels and their split-K
// pairs (kernels/shared_mask_batched_triton_min_runtime.py:814-874, 1150-1216, 1956-1988).
#include "bas_kernels.cuh"

#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

namespace bas {

namespace {

constexpr int kUmmaThreads = 64 + 128;
constexpr int kEpiThreads = 128;
constexpr int kTmemCols = 128;  // two accumulator buffers of 64 fp32 columns

template <int BPAD>
struct UmmaCfg {
  static constexpr int kXTileBytes = BPAD * 128;  // multiple of 1024 for BPAD in {16,32,48,64}
  static constexpr int kStageBytes = kTileBytes + kXTileBytes;
  static constexpr int kStagesRaw = (192 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
};

struct UmmaSmemHeader {
  uint64_t full[16];
  uint64_t empty[16];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t fix_bar;
  uint32_t tmem_base;
  int scan[34];
  int abort_flag;
  int last_flag;
};

__host__ __device__ inline size_t umma_ids_bytes(int nb) { return ((size_t)nb * 2 + 127) / 128 * 128; }

template <int BPAD>
size_t umma_smem_bytes(int nb) {
  return 1024 /*alignment slack*/ + (sizeof(UmmaSmemHeader) + 127) / 128 * 128 + umma_ids_bytes(nb) + 1024 +
         (size_t)UmmaCfg<BPAD>::kStages * UmmaCfg<BPAD>::kStageBytes;
}

template <int BPAD>
__global__ void __launch_bounds__(kUmmaThreads, 1)
    umma_splitk_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap) {
  using Cfg = UmmaCfg<BPAD>;
  constexpr int S = Cfg::kStages;
  constexpr uint32_t kIdesc = umma_idesc_f16(128, BPAD);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sp = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  UmmaSmemHeader* hdr = (UmmaSmemHeader*)sp;
  sp += (sizeof(UmmaSmemHeader) + 127) / 128 * 128;
  uint16_t* s_ids = (uint16_t*)sp;
  sp += umma_ids_bytes(p.nb);
  uint8_t* s_stage = (uint8_t*)(((uintptr_t)sp + 1023) & ~(uintptr_t)1023);  // swizzle atoms need 1 KiB alignment

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &hdr->abort_flag;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&hdr->acc_full[a], 1);
      mbar_init(&hdr->acc_empty[a], kEpiThreads / 32);
    }
    mbar_init(&hdr->fix_bar, kEpiThreads / 32);
    hdr->abort_flag = 0;
    hdr->last_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&xmap);
  }
  if (warp == 2) {
    tmem_alloc(&hdr->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  // Nothing above touches global memory.  The id list may be the previous kernel's output unless
  // the caller declared it stable; X, the workspace and Y always wait.
  const bool early_ids = (p.flags & kFlagStableIds) != 0 && p.count_dev == nullptr;
  if (!early_ids) pdl_wait();
  const int k_act = stage_active_ids(p.ids, p.count_dev, p.k_host, p.bitmap, p.nb, s_ids, hdr->scan, p.status);
  pdl_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = hdr->tmem_base;

  const long long total = (long long)k_act * p.nt;
  // Never more ranges than units: every participating CTA then owns at least one unit, so the
  // contributors of a column tile are a contiguous run of CTAs.
  const int c = blockIdx.x, G = (int)max(1LL, min((long long)gridDim.x, total));
  const long long u0 = (k_act > 0 && c < G) ? part_begin(c, total, G) : 0;
  const long long u1 = (k_act > 0 && c < G) ? part_begin(c + 1, total, G) : 0;
  const int cnt = (int)(u1 - u0);
  int issued = 0;  // tiles whose copies the producer thread has started

  if (k_act == 0) {
    if (early_ids) pdl_wait();
    zero_output(p.y, p.batch, p.n, p.ldy);
  } else if (cnt > 0) {
    if (warp == 0) {
      // ------------------------------ producer (one thread) ------------------------------
      if (lane == 0) {
        int m = 0, n0 = 0;
        if (early_ids) {
          // The ids are not the previous kernel's output: stream the first ring-full of weight
          // tiles while that kernel is still draining, then wait for it before loading X.
          int ahead = 0;
          for (int n = 0; n < cnt && ahead < S; ++n) {
            const long long u = u0 + n;
            const int t = (int)(u / k_act), j = s_ids[(int)(u - (long long)t * k_act)];
            if (j == kSkipId) continue;
            mbar_arrive_expect_tx(&hdr->full[ahead], kTileBytes + Cfg::kXTileBytes);
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
            tma_load_2d(s_stage + (size_t)m * Cfg::kStageBytes + kTileBytes, &xmap, j * kBlockK, 0, &hdr->full[m]);
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
          uint8_t* st = s_stage + (size_t)s * Cfg::kStageBytes;
          mbar_arrive_expect_tx(&hdr->full[s], kTileBytes + Cfg::kXTileBytes);
          bulk_copy_g2s(st, p.packed + ((size_t)j * p.nt + t) * kTileBytes, kTileBytes, &hdr->full[s]);
          tma_load_2d(st + kTileBytes, &xmap, j * kBlockK, 0, &hdr->full[s]);
          issued = ++m;
        }
      }
    } else if (warp == 1) {
      // ------------------------------ MMA issuer (one thread) ------------------------------
      if (lane == 0) {
        int seg = 0, m = 0;
        bool fresh = true;      // the next MMA overwrites the accumulator instead of adding to it
        bool any = false;       // this segment has issued at least one MMA
        for (int n = 0; n < cnt; ++n) {
          const long long u = u0 + n;
          const int i = (int)(u % k_act);
          const int a = seg & 1;
          const bool skip = s_ids[i] == kSkipId;
          const bool last_of_seg = (i == k_act - 1 || n == cnt - 1);
          if (!skip) {
            const int s = m % S;
            bool ok = true;
            if (fresh && seg >= 2) ok = mbar_wait(&hdr->acc_empty[a], ((seg >> 1) - 1) & 1, abort_flag);
            if (ok) ok = mbar_wait(&hdr->full[s], (m / S) & 1, abort_flag);
            if (!ok) {
              atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
              hdr->abort_flag = 1;
              break;
            }
            tc_fence_after_sync();
            const uint32_t st = smem_u32(s_stage + (size_t)s * Cfg::kStageBytes);
            const uint64_t adesc = umma_desc_kmajor_sw128(st);
            const uint64_t bdesc = umma_desc_kmajor_sw128(st + kTileBytes);
            const uint32_t d = tmem_base + (uint32_t)(a * 64);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              // 16 channels = 32 bytes along K: +2 in the descriptor's 16-byte address units
              umma_f16_ss(d, adesc + (uint64_t)(2 * ks), bdesc + (uint64_t)(2 * ks), kIdesc, (fresh && ks == 0) ? 0u : 1u);
            }
            umma_commit(&hdr->empty[s]);  // the stage is free once these MMAs have read it
            fresh = false;
            any = true;
            ++m;
          }
          if (last_of_seg) {
            // A segment made only of skipped units issues no MMA: the epilogue (which checks the
            // id list itself) then takes zeros instead of reading an accumulator nobody wrote.
            if (any) {
              umma_commit(&hdr->acc_full[a]);
            } else {
              if (seg >= 2 && !mbar_wait(&hdr->acc_empty[a], ((seg >> 1) - 1) & 1, abort_flag)) {
                atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
                hdr->abort_flag = 1;
                break;
              }
              mbar_arrive(&hdr->acc_full[a]);
            }
            ++seg;
            fresh = true;
            any = false;
          }
        }
      }
    } else {
      // ------------------------------ epilogue: 4 warps, one TMEM lane quarter each ------------------------------
      const int q = warp & 3;               // a warp may only read TMEM lanes [32*(warp%4), +32)
      const int r = q * 32 + lane;          // row of the tile = output column within the tile
      const int t_first = (int)(u0 / k_act);
      uint32_t fix_phase = 0;
      int seg = 0;
      long long us = u0;
      bool ok = true;
      if (early_ids) pdl_wait();            // before the first write to the workspace or Y
      while (us < u1 && ok) {
        const int t = (int)(us / k_act);
        const long long ue = min(u1, (long long)(t + 1) * k_act);
        const int i0 = (int)(us - (long long)t * k_act), i1 = (int)(ue - (long long)t * k_act);
        const int a = seg & 1;
        if (!mbar_wait(&hdr->acc_full[a], (seg >> 1) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        float v[BPAD];
        bool has_data = false;
        for (int i = i0 + lane; i < i1; i += 32) has_data |= (s_ids[i] != kSkipId);
        has_data = __any_sync(0xffffffffu, has_data);
        if (has_data) {
#pragma unroll
          for (int cc = 0; cc < BPAD / 16; ++cc) {
            uint32_t regs[16];
            tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * 64 + cc * 16), regs);
#pragma unroll
            for (int e = 0; e < 16; ++e) v[cc * 16 + e] = __uint_as_float(regs[e]);
          }
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int b = 0; b < BPAD; ++b) v[b] = 0.f;
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->acc_empty[a]);
        const bool complete = (i0 == 0) && (i1 == k_act);
        ok = store_or_combine<BPAD>(v, p.batch, p.y, p.ldy, p.n, p.partials, p.counters, t, t_first, complete, c, G,
                                    k_act, total, r, lane, &hdr->fix_bar, fix_phase, &hdr->last_flag, abort_flag);
        ++seg;
        us = ue;
      }
      if (!ok) {
        atomicOr(p.status, BAS_DEV_WAIT_EXPIRED);
        hdr->abort_flag = 1;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (hdr->abort_flag != 0 && tid == 0) {
    // Gave up somewhere: do not leave while copies may still be landing in this CTA's memory.
    int zero = 0;
    for (int n = max(0, issued - S); n < issued; ++n) (void)mbar_wait(&hdr->full[n % S], (n / S) & 1, &zero);
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// host side: tensor maps for X and the launch
// ---------------------------------------------------------------------------------------------
struct MapKey {
  const void* x;
  long long ldx;
  int batch, k, bpad;
  bool operator==(const MapKey& o) const {
    return x == o.x && ldx == o.ldx && batch == o.batch && k == o.k && bpad == o.bpad;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& m) const {
    size_t h = (size_t)m.x;
    h = h * 1000003u ^ (size_t)m.ldx;
    h = h * 1000003u ^ (size_t)m.batch;
    h = h * 1000003u ^ (size_t)m.k;
    return h * 1000003u ^ (size_t)m.bpad;
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

// X[batch, K] fp16, row stride ldx: inner dimension K, box {64 channels, bpad rows}, 128-byte swizzle.
cudaError_t get_x_tensor_map(const GemmParams& p, int bpad, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{p.x, p.ldx, p.batch, p.k, bpad};
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
  const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(p.x), gdim, gstride, box, estr,
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

template <int BPAD>
cudaError_t launch_umma_b(const GemmParams& p, int sm_count, cudaStream_t stream) {
  const size_t smem = umma_smem_bytes<BPAD>(p.nb);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(umma_splitk_kernel<BPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  CUtensorMap xmap;
  cudaError_t e = get_x_tensor_map(p, BPAD, &xmap);
  if (e != cudaSuccess) return e;
  const long long units = (long long)(p.bitmap != nullptr ? p.nb : p.k_host) * p.nt;
  const int grid = (int)(units < sm_count ? (units < 1 ? 1 : units) : sm_count);
  count_launch();
  return launch_with_pdl(umma_splitk_kernel<BPAD>, grid, kUmmaThreads, smem, stream, p, xmap);
}

}  // namespace

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
