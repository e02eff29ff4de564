// Weight prepack, bitmap build and the per-step batch-shared mask selection.
#include "bas_kernels.cuh"

#include <atomic>

namespace bas {

namespace {

// ---------------------------------------------------------------------------------------------
// Prepack: W[N, K] (row stride ldw) -> [nb][npad][64] fp16: block j holds, for every output column
// n (padded to a multiple of 8 with zero rows), its 64 channels as one 128-byte row whose 16-byte
// chunk q is stored at chunk position q ^ (n % 8).  Any range of columns of a block is therefore one
// contiguous, already swizzled chunk.  One CTA per (128 columns, block).  Off the hot path (once per
// weight), like the reference's _get_prepacked_weight_block_major
// (kernels/shared_mask_batched_triton_min_runtime.py:3133-3163).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) pack_weight_kernel(const __half* __restrict__ w, int n, int k, long long ldw,
                                                          uint8_t* __restrict__ packed, int npad) {
  const int t = blockIdx.x, j = blockIdx.y;
  const bool vec_ok = ((ldw & 7) == 0) && ((((uintptr_t)w) & 15) == 0);
  for (int idx = threadIdx.x; idx < kTileN * 8; idx += blockDim.x) {
    const int r = idx >> 3, q = idx & 7;
    const int row = t * kTileN + r, col = j * kBlockK + q * 8;
    if (row >= npad) continue;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < n && col < k) {
      const __half* src = w + (size_t)row * ldw + col;
      if (vec_ok && col + 8 <= k) {
        v = *(const uint4*)src;
      } else {
        __half h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = (col + e < k) ? src[e] : __float2half_rn(0.f);
        v = *(const uint4*)h;
      }
    }
    *(uint4*)(packed + ((size_t)j * npad + row) * kRowBytes + ((q ^ (row & 7)) << 4)) = v;
  }
}

// ---------------------------------------------------------------------------------------------
// Bitmap: u8[nb], 1 at active ids (kernels/shared_mask_batched_triton_min_runtime.py:1056-1061).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) build_bitmap_kernel(const int32_t* __restrict__ ids,
                                                           const int32_t* __restrict__ count_dev, int k_host, int nb,
                                                           uint8_t* __restrict__ bitmap) {
  // single CTA: clear, then set
  for (int i = threadIdx.x; i < nb; i += blockDim.x) bitmap[i] = 0;
  __syncthreads();
  int cnt = k_host;
  if (count_dev != nullptr) cnt = min(max(*count_dev, 0), k_host);
  for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
    const int id = ids[i];
    if (id >= 0 && id < nb) bitmap[id] = 1;
  }
}

// ---------------------------------------------------------------------------------------------
// Selection.  Phase 1 (all CTAs): per-(batch row, block) energy in fp64 from exact fp16 squares,
// optional sqrt, batch-summed in row order -> ws_scores[nb].  Phase 2 (the last CTA to finish):
// rank every block by (score descending, id ascending), keep the first n_keep (top-k) or the
// shortest prefix reaching the energy budget, and write the kept ids in ascending order.
// Restates scripts/bench_roundrobin_e2e_decode.py:90-113 and
// scripts/bench_alpaca_energy_budget_e2e.py:43-62 in one launch without host synchronisation.
// ---------------------------------------------------------------------------------------------
constexpr int kSelThreads = 1024;                    // largest block size; the launch picks 256 or 1024
constexpr int kSelBlocksPerCta = 2;                  // activation blocks scored per CTA
constexpr int kSelMaxBatch = 1024;

__global__ void __launch_bounds__(kSelThreads) select_kernel(const SelectParams p) {
  extern __shared__ double s_dyn[];   // phase 1: [kSelBlocksPerCta][batch]; phase 2: scores[nb] + ranks
  __shared__ int s_last;
  __shared__ int s_warp_cnt[kSelThreads / 32];
  __shared__ int s_keep;

  // Launched with programmatic stream serialization: everything this kernel reads (X) or writes
  // (ids, count, byte map, workspace) may still be in use by the kernel before it, so the wait comes
  // first; the kernel after it may be set up meanwhile and waits for this grid's completion itself.
  // With BAS_SCORE_INPUTS_STABLE the caller has promised that the preceding kernel neither writes X nor
  // touches this call's outputs and workspace: scoring and ranking then run beside that kernel (on SMs
  // it leaves free), and the wait moves to just before the outputs are written.
  if (!p.inputs_stable) pdl_wait();
  pdl_launch_dependents();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nthreads = (int)blockDim.x;   // 256 for small batches, 1024 for large ones (measured)
  const int j0 = blockIdx.x * kSelBlocksPerCta;
  const int nj = min(kSelBlocksPerCta, p.nb - j0);

  // ---- phase 1: 8 lanes per (row, block) pair, 16 bytes per lane ----
  const int sub = tid & 7, grp = tid >> 3;           // 32 groups of 8 lanes
  const int pairs = nj * p.batch;
  for (int base = 0; base < pairs; base += nthreads / 8) {
    const int pr = base + grp;
    double e = 0.0;
    if (pr < pairs) {
      const int jj = pr / p.batch, b = pr - jj * p.batch;
      const uint4 v = __ldg((const uint4*)(p.x + (size_t)b * p.ldx + (size_t)(j0 + jj) * kBlockK) + sub);
      if (p.chan_scale != nullptr) {
        // weighted squares: sum_i x_i^2 * scale_i (scripts/bench_roundrobin_e2e_decode.py:106-108)
        const float4* scp = (const float4*)(p.chan_scale + (size_t)(j0 + jj) * kBlockK) + 2 * sub;
        const float4 s0 = __ldg(scp), s1 = __ldg(scp + 1);
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const unsigned int* wds = (const unsigned int*)&v;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          double lo, hi;
          if (p.bf16) {
            lo = (double)__uint_as_float(wds[q] << 16);
            hi = (double)__uint_as_float(wds[q] & 0xffff0000u);
          } else {
            const float2 f = __half22float2(*(const __half2*)&wds[q]);
            lo = (double)f.x;
            hi = (double)f.y;
          }
          e += (lo * lo) * (double)sc[2 * q];
          e += (hi * hi) * (double)sc[2 * q + 1];
        }
      } else if (p.bf16) {
        const unsigned int* wds = (const unsigned int*)&v;
#pragma unroll
        for (int q = 0; q < 4; ++q) {   // a bf16 is the upper half of an fp32; squares are taken in fp64 (range)
          const double lo = (double)__uint_as_float(wds[q] << 16), hi = (double)__uint_as_float(wds[q] & 0xffff0000u);
          e += lo * lo;
          e += hi * hi;
        }
      } else {
        const __half2* h = (const __half2*)&v;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __half22float2(h[q]);
          e += (double)(f.x * f.x);   // a product of two fp16 values is exact in fp32
          e += (double)(f.y * f.y);
        }
      }
    }
    e += __shfl_xor_sync(0xffffffffu, e, 1);
    e += __shfl_xor_sync(0xffffffffu, e, 2);
    e += __shfl_xor_sync(0xffffffffu, e, 4);
    if (pr < pairs && sub == 0) {
      const int jj = pr / p.batch, b = pr - jj * p.batch;
      s_dyn[jj * p.batch + b] = (p.score_kind == BAS_SCORE_NORM) ? sqrt(e) : e;
    }
  }
  __syncthreads();
  if (tid < nj) {
    double s = 0.0;
    for (int b = 0; b < p.batch; ++b) s += s_dyn[tid * p.batch + b];   // batch rows in order
    s = s / (double)p.batch;
    if (p.block_mult != nullptr) s *= (double)__ldg(p.block_mult + j0 + tid);
    p.ws_scores[j0 + tid] = s;
    __threadfence();
  }
  __syncthreads();
  if (tid == 0) {
    const unsigned int old = atomicAdd(p.ws_done, 1u);
    s_last = (old == gridDim.x - 1) ? 1 : 0;
    if (s_last) *p.ws_done = 0u;   // re-arm for the next call
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  // ---- phase 2: one CTA ranks all blocks ----
  double* s_score = s_dyn;                              // [nb]
  unsigned long long* s_key = (unsigned long long*)(s_dyn + p.nb);   // [nb] ranking keys (score_key)
  int* s_rank = (int*)(s_key + p.nb);                   // [nb]
  int* s_order = s_rank + p.nb;                         // [nb] block id at each rank (budget mode)
  for (int j = tid; j < p.nb; j += nthreads) {
    const double s = __ldcg(p.ws_scores + j);
    s_score[j] = s;
    s_key[j] = score_key(s);
  }
  __syncthreads();
  // one thread per block counts the blocks that rank before it (about 30 k comparisons in all: the
  // instruction issue of one SM bounds this step at roughly 0.8 us whatever the thread count).
  // Keys are totally ordered (NaN ranks first, like torch.topk), so the ranks are a permutation.
  for (int j = tid; j < p.nb; j += nthreads) {
    const unsigned long long sj = s_key[j];
    int rank = 0;
    for (int i = 0; i < p.nb; ++i) {
      const unsigned long long si = s_key[i];
      rank += (si > sj || (si == sj && i < j)) ? 1 : 0;
    }
    s_rank[j] = rank;
    s_order[rank] = j;
  }
  __syncthreads();
  if (tid == 0) {
    int keep = p.n_keep;
    if (p.mode == 1) {
      // energy budget: shortest descending prefix whose sum reaches energy_keep of the total (a total
      // that is not a number keeps every block)
      double total = 0.0;
      for (int r = 0; r < p.nb; ++r) total += s_score[s_order[r]];
      const double thresh = p.energy_keep * total;
      double cum = 0.0;
      int kk = p.nb;
      for (int r = 0; r < p.nb; ++r) {
        cum += s_score[s_order[r]];
        if (cum >= thresh) { kk = r + 1; break; }
      }
      keep = max(p.n_keep, min(p.nb, kk));
      if (keep > p.full_above) keep = p.nb;   // too little would be skipped: run every block
    }
    s_keep = min(max(keep, 0), p.nb);
  }
  __syncthreads();
  const int keep = s_keep;
  // Stable inputs: everything so far ran beside the preceding kernel and wrote only the workspace and
  // shared memory.  The caller's outputs are written after that kernel has completed; as this CTA is
  // part of the grid, the grid also completes after it, which keeps completions in stream order.
  if (p.inputs_stable) pdl_wait();
  // ascending compaction of the kept ids
  int running = 0;
  for (int base = 0; base < p.nb; base += nthreads) {
    const int j = base + tid;
    const bool kept = (j < p.nb) && (s_rank[j] < keep);
    if (j < p.nb && p.scores_out != nullptr) p.scores_out[j] = s_score[j];
    if (j < p.nb && p.bitmap_out != nullptr) p.bitmap_out[j] = kept ? 1 : 0;
    const unsigned m = __ballot_sync(0xffffffffu, kept);
    if (lane == 0) s_warp_cnt[warp] = __popc(m);
    __syncthreads();
    int off = running;
    for (int w = 0; w < warp; ++w) off += s_warp_cnt[w];
    const int pos = off + __popc(m & ((1u << lane) - 1u));
    if (kept && pos < keep) p.ids_out[pos] = j;
    for (int w = 0; w < nthreads / 32; ++w) running += s_warp_cnt[w];
    __syncthreads();
  }
  if (tid == 0) *p.count_out = keep;
}

}  // namespace

cudaError_t launch_pack(const __half* w, int n, int k, long long ldw, uint8_t* packed, cudaStream_t stream) {
  const int nb = (k + kBlockK - 1) / kBlockK, npad = padded_cols(n), nt = (npad + kTileN - 1) / kTileN;
  pack_weight_kernel<<<dim3(nt, nb), 256, 0, stream>>>(w, n, k, ldw, packed, npad);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_build_bitmap(const int32_t* ids, const int32_t* count_dev, int k_host, int nb, uint8_t* bitmap,
                                cudaStream_t stream) {
  build_bitmap_kernel<<<1, 256, 0, stream>>>(ids, count_dev, k_host, nb, bitmap);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_select(const SelectParams& p, int sm_count, cudaStream_t stream) {
  (void)sm_count;
  if (p.batch > kSelMaxBatch) return cudaErrorInvalidValue;
  const int grid = (p.nb + kSelBlocksPerCta - 1) / kSelBlocksPerCta;
  const size_t phase1 = sizeof(double) * kSelBlocksPerCta * (size_t)p.batch;
  const size_t phase2 = (2 * sizeof(double) + 2 * sizeof(int)) * (size_t)p.nb;
  const size_t smem = phase1 > phase2 ? phase1 : phase2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) return e;
    if (smem > 96 * 1024) return cudaErrorInvalidValue;
  }
  count_launch();
  // 1024 threads score 128 (block, row) pairs per round instead of 32: pays from about 32 rows
  return launch_with_pdl(select_kernel, grid, p.batch >= 32 ? kSelThreads : 256, smem, 1, stream, p);
}

}  // namespace bas

// ---------------------------------------------------------------------------------------------
// Selection without any allocation: the kernel's scratch (per-block scores + the arrival counter)
// lives in a fixed device array that is part of the library image.  See bas_select_topk_noalloc in
// include/bas.h for who needs this and what it costs.
// ---------------------------------------------------------------------------------------------
namespace bas {
namespace {
// [0,256): arrival counter (first word), [256, ...): one fp64 score per activation block.
static __device__ __align__(256) unsigned char g_select_scratch[256 + sizeof(double) * BAS_NOALLOC_MAX_BLOCKS];
}  // namespace
}  // namespace bas

extern "C" BAS_API int bas_select_topk_noalloc(const void* x_dev, int64_t ldx, int batch, int k, int n_keep,
                                               int score_kind, int32_t* ids_out_dev, int32_t* count_out_dev,
                                               uint8_t* bitmap_out_dev, double* scores_out_dev, void* stream) {
  using namespace bas;
  if (x_dev == nullptr || ids_out_dev == nullptr || count_out_dev == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  if (batch <= 0 || k < kBlockK || ldx < k || (((uintptr_t)x_dev) & 15u) != 0 || (ldx & 7) != 0)
    return BAS_ERR_INVALID_ARGUMENT;
  const int nb = k / kBlockK;
  if (nb > BAS_NOALLOC_MAX_BLOCKS) return BAS_ERR_TOO_LARGE;   // the fixed scratch holds no more scores
  const int bf16 = (score_kind & BAS_SCORE_BF16) != 0 ? 1 : 0;
  score_kind &= ~BAS_SCORE_BF16;
  if (score_kind != BAS_SCORE_NORM && score_kind != BAS_SCORE_ENERGY) return BAS_ERR_INVALID_ARGUMENT;
  if (n_keep < 0 || n_keep > nb) return BAS_ERR_INVALID_ARGUMENT;
  if (batch > kSelMaxBatch) return BAS_ERR_UNSUPPORTED;   // before anything is enqueued

  // In host code the array's name is only a handle; the device address has to be asked for, once per
  // device, with that device current.  The first call on a device does this (any thread may be first:
  // the cache entries are atomic, and every thread that looks the address up gets the same answer).
  static std::atomic<void*> scratch_addr[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (dev < 0 || dev >= 64) return BAS_ERR_UNSUPPORTED;
  void* scratch = scratch_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    e = cudaGetSymbolAddress(&scratch, g_select_scratch);
    if (e != cudaSuccess || scratch == nullptr) return record_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
    scratch_addr[dev].store(scratch, std::memory_order_release);
  }
  cudaStream_t s = (cudaStream_t)stream;
  // The array keeps whatever the previous call left: the arrival counter must start at zero.
  e = cudaMemsetAsync(scratch, 0, 256, s);
  if (e != cudaSuccess) return record_cuda_error(e);

  SelectParams p;
  p.x = (const __half*)x_dev;
  p.ldx = (long long)ldx;
  p.batch = batch;
  p.k = k;
  p.nb = nb;
  p.mode = 0;
  p.n_keep = n_keep;
  p.score_kind = score_kind;
  p.bf16 = bf16;
  p.energy_keep = 0.0;
  p.ids_out = ids_out_dev;
  p.count_out = count_out_dev;
  p.bitmap_out = bitmap_out_dev;
  p.scores_out = scores_out_dev;
  p.ws_done = (unsigned int*)scratch;
  p.ws_scores = (double*)((unsigned char*)scratch + 256);
  e = launch_select(p, 0, s);
  return e == cudaSuccess ? BAS_OK : record_cuda_error(e);
}
