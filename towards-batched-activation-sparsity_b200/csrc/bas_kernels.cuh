// Kernel launch parameters shared by the two contraction kernels and their host launchers.
#pragma once

#include "bas_common.cuh"

namespace bas {

// Exchange area of a row-parallel contraction whose sum over the ranks of one box is formed inside
// the kernel.  Every rank owns one area (device memory mapped into its peers); all areas have the
// same layout:
//   [0, kTpHeaderBytes)      private to the owner: word 0 = exchange calls completed, word 1 = CTAs
//                            of the current call that have finished
//   [kTpHeaderBytes, ...)    two receive buffers, used alternately; each holds, per source rank, a
//                            [rows][ldp] array of 8-byte words {fp32 partial, call number}
// A rank writes its partial straight into every rank's receive buffer (its own included) with single
// 64-bit stores: a word whose upper half equals the current call number is valid, so no flag, fence
// or second round trip is needed - the reader polls its own memory.
constexpr int kTpMaxRanks = 8;
constexpr int kTpHeaderBytes = 256;
struct TpExchange {
  int world;                           // 0: no exchange, the kernel stores Y itself
  int rank;
  int ldp;                             // row stride of a receive array, in words
  long long src_words;                 // words per source rank in one receive buffer (= max rows * ldp)
  unsigned char* area[kTpMaxRanks];    // every rank's area as mapped here
  unsigned char* own;                  // == area[rank]
  long long sel_words;                 // where the block scores of a sharded selection land, in words from the area's start
};
// Behind the receive buffers: two 64-bit words per activation block, {stamp, upper half of the score} and
// {stamp, lower half}, written by the rank that holds the block into every rank's area (list launches with
// selection entries over K-sharded activations); header word 2 counts such entries completed.
constexpr int kTpSelBlocks = 1024;
constexpr size_t kTpSelBytes = (size_t)kTpSelBlocks * 2 * 8;

// Mask selection run inside the contraction kernel (cluster modes only): every cluster scores all
// blocks of X, its CTAs sharing the blocks and exchanging the scores through shared memory, ranks them
// and compacts the kept ids straight into the id list the contraction then walks.
struct FusedSelect {
  int mode;            // 0 = off (ids / byte map given), 1 = top-k, 2 = energy budget
  int n_keep;          // top-k: blocks to keep; budget: minimum to keep
  int score_kind;      // BAS_SCORE_NORM / BAS_SCORE_ENERGY
  int nb_sel;          // K / 64 rounded down: trailing channels are never scored
  double energy_keep;  // budget mode
  int32_t* ids_out;    // optional outputs, written by CTA 0 only
  int32_t* count_out;
  uint8_t* bitmap_out;
  double* scores_out;
};

struct GemmParams {
  const __half* x;          // [batch, K], row stride ldx
  long long ldx;
  const uint8_t* packed;    // [nb][npad][64] fp16, 16-byte chunks of row n stored at chunk q ^ (n % 8)
  const int32_t* ids;       // active block ids (or null when bitmap is given)
  const int32_t* count_dev; // optional device-side number of ids
  int k_host;               // number of ids (upper bound when count_dev is given)
  const uint8_t* bitmap;    // optional byte map [nb]
  int batch, k, n, nb;
  int npad;                 // n rounded up to a multiple of 8 (rows of the packed layout)
  int ranges;               // column ranges = CTAs (clusters) of the grid
  int cluster;              // CTAs per cluster splitting the active blocks of one range (1, 2 or 4)
  int stages;               // ring slots
  int group;                // blocks per ring slot: one barrier hand-off covers this many chunks
  int wslot;                // bytes reserved per slot for a weight chunk (multiple of 1024)
  int issuers;              // MMA-issuing warps in use (2 or 4), each with its own accumulators
  int tile_cols;            // output columns one pass of a CTA covers (128)
  __half* y;                // [batch, N], row stride ldy
  long long ldy;
  int flags;                // kFlag* bits
  unsigned int* status;     // workspace: status word
  long long wait_cycles;    // bound of every wait of the kernel (bas_set_wait_ms)
  TpExchange tp;            // row-parallel sum over ranks (world 0 = off)
  FusedSelect sel;          // mask selection inside the kernel (mode 0 = off)
#ifdef BAS_TRACE
  long long* trace;         // diagnostic build only: per-role cycle counters of CTA 0
#endif
};

constexpr int kFlagStableIds = 16;   // BAS_GEMM_IDS_STABLE: the id list is not written by the previous kernel
constexpr int kFlagStableX = 64;     // BAS_GEMM_X_STABLE: nor is X (only with kFlagStableIds)
constexpr int kFlagLateWait = 1 << 25;   // set by the launcher (stable X, grid of at most half the SMs): wait for the predecessor only at the stores
constexpr int kFlagMultiAcc = 1 << 26;   // set by the launcher: every 128-column pass of a CTA has accumulator columns of its own
constexpr int kFlagNextIndependent = 128;   // BAS_GEMM_NEXT_INDEPENDENT: the next call can run beside this one (grid-size hint)
constexpr int kFlagBf16 = 32;        // BAS_GEMM_BF16: X, W and Y are bfloat16 (same 16-bit containers)

// Launch with the programmatic-serialization attribute, so that this kernel's preamble (and, when
// the ids are stable, its weight copies) may overlap the tail of the previous kernel in the stream.
// BAS_PDL=0 in the environment turns the attribute off.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_with_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, int cluster,
                            cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (cluster > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Host launchers (defined next to their kernels).  `sm_count` is the persistent grid's upper bound.
cudaError_t launch_gemv(const GemmParams& p, int sm_count, cudaStream_t stream);
cudaError_t launch_umma(const GemmParams& p, int sm_count, cudaStream_t stream);
cudaError_t launch_pack(const __half* w, int n, int k, long long ldw, uint8_t* packed, cudaStream_t stream);
inline int padded_cols(int n) { return (n + 7) / 8 * 8; }
cudaError_t launch_build_bitmap(const int32_t* ids, const int32_t* count_dev, int k_host, int nb, uint8_t* bitmap,
                                cudaStream_t stream);

struct SelectParams {
  const __half* x;
  long long ldx;
  int batch, k, nb;
  int mode;           // 0 = top-k, 1 = energy budget
  int n_keep;         // top-k: blocks to keep; budget: min_keep
  int score_kind;     // BAS_SCORE_NORM / BAS_SCORE_ENERGY
  int bf16;           // x holds bfloat16 instead of fp16
  double energy_keep; // budget mode
  int32_t* ids_out;
  int32_t* count_out;
  uint8_t* bitmap_out;
  double* scores_out;
  double* ws_scores;      // workspace: [nb] fp64 batch-summed scores
  unsigned int* ws_done;  // workspace: CTA arrival counter
  const float* chan_scale = nullptr;   // optional [64 * nb]: per-channel weight of the squares (16-byte aligned)
  const float* block_mult = nullptr;   // optional [nb]: factor on the batch-mean score
  int full_above = 0x7fffffff;   // budget mode: a kept count above this keeps every block (the dense fallback)
  int inputs_stable = 0;   // BAS_SCORE_INPUTS_STABLE: score at once, wait for the preceding kernel only before leaving
};
cudaError_t launch_select(const SelectParams& p, int sm_count, cudaStream_t stream);

void count_launch(int n = 1);
// Bound, in clock64 ticks, that launches take for their waits (about one second unless bas_set_wait_ms changed it).
long long wait_cycles_now();
// Remembers a failed CUDA call for bas_last_cuda_error() on this thread; returns BAS_ERR_CUDA.
int record_cuda_error(cudaError_t e);
// cuTensorMapEncodeTiled of the loaded driver as an untyped pointer (null if unavailable).
void* tensor_map_encoder();

}  // namespace bas

// One rank's view of a tensor-parallel group's exchange areas (bas_tp_* in bas_api.cu; the list kernel's
// host side reads it too).
struct bas_tp {
  int rank = 0, world = 0, max_batch = 0, n = 0, npad = 0;
  size_t bytes = 0;
  unsigned char* area[bas::kTpMaxRanks] = {};   // area[rank] is this rank's own allocation
  bool opened[bas::kTpMaxRanks] = {};
};
