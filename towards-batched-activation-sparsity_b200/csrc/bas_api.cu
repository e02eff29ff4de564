// The C ABI of libbas: argument checks, workspace carving, kernel-family choice and the host-buffer
// operator.  See include/bas.h for the contract of every entry point.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "bas_kernels.cuh"

namespace bas {

#ifdef BAS_TRACE
static long long* g_trace_dev = nullptr;   // diagnostic build only
#endif

static std::atomic<unsigned long long> g_launches{0};
static thread_local int g_last_cuda_error = 0;

static std::atomic<long long> g_wait_cycles{kWaitCycles};
long long wait_cycles_now() { return g_wait_cycles.load(std::memory_order_relaxed); }

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("BAS_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

int record_cuda_error(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return BAS_ERR_CUDA;
}

namespace {

int cuda_fail(cudaError_t e) { return record_cuda_error(e); }

struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
};

// Per-device facts, read once.
int device_info(DeviceInfo* out) {
  static DeviceInfo cache[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return BAS_ERR_UNSUPPORTED;
  if (!ready[dev].load(std::memory_order_acquire)) {
    DeviceInfo d;
    e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    cache[dev] = d;
    ready[dev].store(1, std::memory_order_release);
  }
  *out = cache[dev];
  return BAS_OK;
}

inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15u) == 0; }

}  // namespace
}  // namespace bas

using namespace bas;

extern "C" {

#ifdef BAS_TRACE
BAS_API int bas_debug_trace(long long* out64, int reset) {
  if (g_trace_dev == nullptr) return 1;
  cudaError_t e = cudaMemcpy(out64, g_trace_dev, sizeof(long long) * 1024, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && reset) e = cudaMemset(g_trace_dev, 0, sizeof(long long) * 1024);
  return e == cudaSuccess ? 0 : 4;
}
#endif

const char* bas_status_string(int status) {
  switch (status) {
    case BAS_OK: return "ok";
    case BAS_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, bad size, misaligned pointer or stride)";
    case BAS_ERR_UNSUPPORTED: return "unsupported size or device (needs sm_100, batch <= 64, K/64 <= 4096)";
    case BAS_ERR_WORKSPACE: return "workspace missing or too small";
    case BAS_ERR_CUDA: return "a CUDA call failed (see bas_last_cuda_error)";
    case BAS_ERR_DEVICE_FLAG: return "a kernel flagged a bad block id or an expired wait";
    case BAS_ERR_TOO_LARGE: return "size beyond the fixed capacity of this entry point";
    default: return "unknown status";
  }
}

int bas_last_cuda_error(void) { return g_last_cuda_error; }

int bas_set_wait_ms(double wait_ms) {
  if (!(wait_ms > 0.0) || wait_ms > 10000.0) return BAS_ERR_INVALID_ARGUMENT;
  g_wait_cycles.store((long long)(wait_ms * 2.0e6), std::memory_order_relaxed);   // clock64 ticks at about 2 GHz
  return BAS_OK;
}

unsigned long long bas_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

size_t bas_packed_weight_bytes(int n, int k) {
  if (n <= 0 || k <= 0) return 0;
  const size_t nb = ((size_t)k + kBlockK - 1) / kBlockK;
  return nb * (size_t)padded_cols(n) * (size_t)kRowBytes;
}

int bas_pack_weight(const void* w_dev, int n, int k, int64_t ldw, void* packed_dev, void* stream) {
  if (w_dev == nullptr || packed_dev == nullptr || n <= 0 || k <= 0 || ldw < k) return BAS_ERR_INVALID_ARGUMENT;
  if (!aligned16(packed_dev)) return BAS_ERR_INVALID_ARGUMENT;
  if ((k + kBlockK - 1) / kBlockK > BAS_MAX_BLOCKS) return BAS_ERR_UNSUPPORTED;
  cudaError_t e = launch_pack((const __half*)w_dev, n, k, (long long)ldw, (uint8_t*)packed_dev, (cudaStream_t)stream);
  return e == cudaSuccess ? BAS_OK : cuda_fail(e);
}

size_t bas_gemm_workspace_bytes(int batch, int n) {
  (void)n;
  if (batch <= 0) return 0;
  return kWsBytes;
}

int bas_workspace_init(void* ws_dev, size_t ws_bytes, void* stream) {
  if (ws_dev == nullptr || ws_bytes == 0) return BAS_ERR_INVALID_ARGUMENT;
  cudaError_t e = cudaMemsetAsync(ws_dev, 0, ws_bytes, (cudaStream_t)stream);
  return e == cudaSuccess ? BAS_OK : cuda_fail(e);
}

// ---------------------------------------------------------------------------------------------
// exchange areas of a tensor-parallel group (one process per GPU, all on one box)
// ---------------------------------------------------------------------------------------------
// (struct bas_tp: bas_kernels.cuh)
static size_t tp_area_bytes(int world, int max_batch, int npad) {
  return (size_t)kTpHeaderBytes + 2 * 8 * (size_t)world * (size_t)max_batch * (size_t)npad + kTpSelBytes;
}

int bas_tp_create(bas_tp** out, int rank, int world, int max_batch, int n) {
  if (out == nullptr || world < 1 || world > kTpMaxRanks || rank < 0 || rank >= world || max_batch <= 0 ||
      max_batch > BAS_MAX_BATCH || n <= 0)
    return BAS_ERR_INVALID_ARGUMENT;
  bas_tp* t = new (std::nothrow) bas_tp();
  if (t == nullptr) return BAS_ERR_CUDA;
  t->rank = rank;
  t->world = world;
  t->max_batch = max_batch;
  t->n = n;
  t->npad = padded_cols(n);
  t->bytes = tp_area_bytes(world, max_batch, t->npad);
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, t->bytes);
  if (e == cudaSuccess) e = cudaMemset(ptr, 0, t->bytes);   // call counters and the words' call numbers start at zero
  if (e != cudaSuccess) {
    if (ptr != nullptr) cudaFree(ptr);
    delete t;
    return cuda_fail(e);
  }
  t->area[rank] = (unsigned char*)ptr;
  *out = t;
  return BAS_OK;
}

int bas_tp_handle(bas_tp* t, void* handle_out) {
  if (t == nullptr || handle_out == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == BAS_TP_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, t->area[t->rank]);
  if (e != cudaSuccess) return cuda_fail(e);
  std::memcpy(handle_out, &h, sizeof(h));
  return BAS_OK;
}

int bas_tp_connect(bas_tp* t, const void* handles) {
  if (t == nullptr || (t->world > 1 && handles == nullptr)) return BAS_ERR_INVALID_ARGUMENT;
  for (int q = 0; q < t->world; ++q) {
    if (q == t->rank || t->opened[q]) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, (const unsigned char*)handles + (size_t)q * BAS_TP_HANDLE_BYTES, sizeof(h));
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(e);
    t->area[q] = (unsigned char*)ptr;
    t->opened[q] = true;
  }
  return BAS_OK;
}

int bas_tp_disconnect(bas_tp* t) {
  if (t == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  cudaError_t first = cudaSuccess;
  for (int q = 0; q < t->world; ++q)
    if (t->opened[q]) {
      cudaError_t e = cudaIpcCloseMemHandle(t->area[q]);
      if (e != cudaSuccess && first == cudaSuccess) first = e;
      t->area[q] = nullptr;
      t->opened[q] = false;
    }
  return first == cudaSuccess ? BAS_OK : cuda_fail(first);
}

void bas_tp_destroy(bas_tp* t) {
  if (t == nullptr) return;
  (void)bas_tp_disconnect(t);
  if (t->area[t->rank] != nullptr) cudaFree(t->area[t->rank]);
  delete t;
}

// `sel` (optional): run the mask selection inside the contraction kernel; ids_dev / count_dev /
// bitmap_dev are then ignored.  Returns BAS_ERR_UNSUPPORTED without launching when the work split of
// this shape has no cluster to run it in.
static int gemm_impl(const bas_tp* tp, const FusedSelect* sel, const void* x_dev, int64_t ldx, const void* packed_dev,
                     const int32_t* ids_dev, const int32_t* count_dev, int k_host, const uint8_t* bitmap_dev, int batch,
                     int k, int n, void* y_dev, int64_t ldy, void* ws_dev, size_t ws_bytes, int flags, void* stream) {
  if (x_dev == nullptr || packed_dev == nullptr || y_dev == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  if (batch <= 0 || k <= 0 || n <= 0 || k_host < 0 || ldx < k || ldy < n) return BAS_ERR_INVALID_ARGUMENT;
  if (batch > BAS_MAX_BATCH) return BAS_ERR_UNSUPPORTED;
  const int nb = (k + kBlockK - 1) / kBlockK;
  if (nb > BAS_MAX_BLOCKS) return BAS_ERR_UNSUPPORTED;
  if (sel == nullptr && bitmap_dev == nullptr && ids_dev == nullptr && k_host > 0) return BAS_ERR_INVALID_ARGUMENT;
  if (k_host > nb) {
    if (bitmap_dev == nullptr) return BAS_ERR_INVALID_ARGUMENT;  // ids are distinct
    k_host = nb;                                                 // with a byte map k_host is only a hint
  }
  // bulk copies: 16-byte aligned rows whose valid length is a multiple of 16 bytes
  if (!aligned16(x_dev) || !aligned16(packed_dev) || (ldx & 7) != 0 || (k & 7) != 0) return BAS_ERR_INVALID_ARGUMENT;
  if (ws_dev == nullptr || ws_bytes < bas_gemm_workspace_bytes(batch, n)) return BAS_ERR_WORKSPACE;
  const int family = flags & 3;
  if (flags < 0 || family > 2 || (flags & ~(3 | BAS_GEMM_IDS_STABLE | BAS_GEMM_X_STABLE | BAS_GEMM_NEXT_INDEPENDENT | BAS_GEMM_BF16 | 0x700 | 0x7000 | 0xff0000 | (1 << 24))) != 0) return BAS_ERR_INVALID_ARGUMENT;

  DeviceInfo di;
  int st = device_info(&di);
  if (st != BAS_OK) return st;
  if (di.cc_major != 10) return BAS_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;

  if (tp != nullptr) {
    for (int q = 0; q < tp->world; ++q)
      if (tp->area[q] == nullptr) return BAS_ERR_INVALID_ARGUMENT;   // bas_tp_connect has not run
    if (batch > tp->max_batch || n > tp->n || family == 1) return BAS_ERR_INVALID_ARGUMENT;
  }
  if (tp == nullptr && sel == nullptr && bitmap_dev == nullptr && k_host == 0) {  // empty active set known on the host: Y = 0
    cudaError_t e = cudaMemset2DAsync(y_dev, (size_t)ldy * 2, 0, (size_t)n * 2, (size_t)batch, s);
    return e == cudaSuccess ? BAS_OK : cuda_fail(e);
  }

  GemmParams p;
  p.x = (const __half*)x_dev;
  p.ldx = (long long)ldx;
  p.packed = (const uint8_t*)packed_dev;
  p.ids = ids_dev;
  p.count_dev = count_dev;
  p.k_host = k_host;
  p.bitmap = bitmap_dev;
  p.batch = batch;
  p.k = k;
  p.n = n;
  p.nb = nb;
  p.npad = padded_cols(n);
  p.ranges = p.cluster = p.stages = p.wslot = 0;   // chosen by the launcher
  p.y = (__half*)y_dev;
  p.ldy = (long long)ldy;
  p.flags = flags;
  p.status = (unsigned int*)ws_dev;
  p.wait_cycles = wait_cycles_now();
  p.sel = FusedSelect{};
  if (sel != nullptr) {
    p.sel = *sel;
    p.ids = nullptr;
    p.count_dev = nullptr;
    p.bitmap = nullptr;
  }
  p.tp = TpExchange{};
  if (tp != nullptr) {
    p.tp.world = tp->world;
    p.tp.rank = tp->rank;
    p.tp.ldp = tp->npad;
    p.tp.src_words = (long long)tp->max_batch * tp->npad;
    p.tp.own = tp->area[tp->rank];
    p.tp.sel_words = 0;
    for (int q = 0; q < tp->world; ++q) p.tp.area[q] = tp->area[q];
  }
#ifdef BAS_TRACE
  if (g_trace_dev == nullptr) {
    cudaMalloc(&g_trace_dev, sizeof(long long) * 1024);
    cudaMemset(g_trace_dev, 0, sizeof(long long) * 1024);
  }
  p.trace = g_trace_dev;
#endif

  const int grid_cap = di.sm_count;
  // Measured on B200, the tcgen05 kernel is the faster one at every batch size (it issues a quarter
  // of the copies per byte), so it is the default; the CUDA-core kernel runs on request.
  const bool small = (family == 1);
  if (small && (batch > 8 || (flags & BAS_GEMM_BF16) != 0)) return BAS_ERR_UNSUPPORTED;   // the CUDA-core kernel is fp16 only
  if (small && sel != nullptr) return BAS_ERR_UNSUPPORTED;
  cudaError_t e = small ? launch_gemv(p, grid_cap, s) : launch_umma(p, grid_cap, s);
  if (e == cudaErrorNotSupported && sel != nullptr) return BAS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? BAS_OK : cuda_fail(e);
}

int bas_gemm_ex(const void* x_dev, int64_t ldx, const void* packed_dev, const int32_t* ids_dev,
                const int32_t* count_dev, int k_host, const uint8_t* bitmap_dev, int batch, int k, int n,
                void* y_dev, int64_t ldy, void* ws_dev, size_t ws_bytes, int flags, void* stream) {
  return gemm_impl(nullptr, nullptr, x_dev, ldx, packed_dev, ids_dev, count_dev, k_host, bitmap_dev, batch, k, n, y_dev,
                   ldy, ws_dev, ws_bytes, flags, stream);
}

int bas_gemm_allreduce(bas_tp* tp, const void* x_dev, int64_t ldx, const void* packed_dev, const int32_t* ids_dev,
                       const int32_t* count_dev, int k_host, const uint8_t* bitmap_dev, int batch, int k, int n,
                       void* y_dev, int64_t ldy, void* ws_dev, size_t ws_bytes, int flags, void* stream) {
  if (tp == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  // calls that exchange partial sums with other ranks stay one deep: the X-stable promise is not used
  return gemm_impl(tp, nullptr, x_dev, ldx, packed_dev, ids_dev, count_dev, k_host, bitmap_dev, batch, k, n, y_dev, ldy,
                   ws_dev, ws_bytes, flags & ~BAS_GEMM_X_STABLE, stream);
}

int bas_gemm(const void* x_dev, int64_t ldx, const void* packed_dev, const int32_t* ids_dev, const int32_t* count_dev,
             int k_host, const uint8_t* bitmap_dev, int batch, int k, int n, void* y_dev, int64_t ldy, void* ws_dev,
             size_t ws_bytes, void* stream) {
  return bas_gemm_ex(x_dev, ldx, packed_dev, ids_dev, count_dev, k_host, bitmap_dev, batch, k, n, y_dev, ldy, ws_dev,
                     ws_bytes, 0, stream);
}

int bas_read_device_status(void* ws_dev, unsigned int* flags_out, void* stream) {
  if (ws_dev == nullptr || flags_out == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(flags_out, ws_dev, sizeof(unsigned int), cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemsetAsync(ws_dev, 0, sizeof(unsigned int), s);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaStreamSynchronize(s);
  return e == cudaSuccess ? BAS_OK : cuda_fail(e);
}

int bas_build_bitmap(const int32_t* ids_dev, const int32_t* count_dev, int k_host, int nb, uint8_t* bitmap_dev,
                     void* stream) {
  if (bitmap_dev == nullptr || nb <= 0 || k_host < 0 || (k_host > 0 && ids_dev == nullptr))
    return BAS_ERR_INVALID_ARGUMENT;
  cudaError_t e = launch_build_bitmap(ids_dev, count_dev, k_host, nb, bitmap_dev, (cudaStream_t)stream);
  return e == cudaSuccess ? BAS_OK : cuda_fail(e);
}

size_t bas_select_workspace_bytes(int k) {
  if (k <= 0) return 0;
  const size_t nb = (size_t)(k / kBlockK);
  return 256 + sizeof(double) * (nb > 0 ? nb : 1);
}

static int select_common(const void* x_dev, int64_t ldx, int batch, int k, int mode, int n_keep, int score_kind,
                         double energy_keep, int32_t* ids_out_dev, int32_t* count_out_dev, uint8_t* bitmap_out_dev,
                         double* scores_out_dev, void* ws_dev, size_t ws_bytes, void* stream,
                         const float* chan_scale_dev = nullptr, const float* block_mult_dev = nullptr,
                         int full_above = 0x7fffffff) {
  if (chan_scale_dev != nullptr && !aligned16(chan_scale_dev)) return BAS_ERR_INVALID_ARGUMENT;
  if (x_dev == nullptr || ids_out_dev == nullptr || count_out_dev == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  if (batch <= 0 || k < kBlockK || ldx < k || !aligned16(x_dev) || (ldx & 7) != 0) return BAS_ERR_INVALID_ARGUMENT;
  const int nb = k / kBlockK;  // trailing K mod 64 channels are never scored (d_eff)
  if (nb > BAS_MAX_BLOCKS) return BAS_ERR_UNSUPPORTED;
  const int bf16 = (score_kind & BAS_SCORE_BF16) != 0 ? 1 : 0;
  const int inputs_stable = (score_kind & BAS_SCORE_INPUTS_STABLE) != 0 ? 1 : 0;
  score_kind &= ~(BAS_SCORE_BF16 | BAS_SCORE_INPUTS_STABLE);
  if (score_kind != BAS_SCORE_NORM && score_kind != BAS_SCORE_ENERGY) return BAS_ERR_INVALID_ARGUMENT;
  if (n_keep < 0 || n_keep > nb) return BAS_ERR_INVALID_ARGUMENT;
  if (ws_dev == nullptr || ws_bytes < bas_select_workspace_bytes(k)) return BAS_ERR_WORKSPACE;
  DeviceInfo di;
  int st = device_info(&di);
  if (st != BAS_OK) return st;
  SelectParams p;
  p.x = (const __half*)x_dev;
  p.ldx = (long long)ldx;
  p.batch = batch;
  p.k = k;
  p.nb = nb;
  p.mode = mode;
  p.n_keep = n_keep;
  p.score_kind = score_kind;
  p.bf16 = bf16;
  p.energy_keep = energy_keep;
  p.ids_out = ids_out_dev;
  p.count_out = count_out_dev;
  p.bitmap_out = bitmap_out_dev;
  p.scores_out = scores_out_dev;
  p.ws_done = (unsigned int*)ws_dev;
  p.ws_scores = (double*)((uint8_t*)ws_dev + 256);
  p.chan_scale = chan_scale_dev;
  p.block_mult = block_mult_dev;
  p.inputs_stable = inputs_stable;
  p.full_above = full_above;
  if (chan_scale_dev != nullptr) p.score_kind = BAS_SCORE_ENERGY;   // weighted squares, no root (as the reference)
  cudaError_t e = launch_select(p, di.sm_count, (cudaStream_t)stream);
  return e == cudaSuccess ? BAS_OK : cuda_fail(e);
}

int bas_select_topk(const void* x_dev, int64_t ldx, int batch, int k, int n_keep, int score_kind, int32_t* ids_out_dev,
                    int32_t* count_out_dev, uint8_t* bitmap_out_dev, double* scores_out_dev, void* ws_dev,
                    size_t ws_bytes, void* stream) {
  return select_common(x_dev, ldx, batch, k, 0, n_keep, score_kind, 0.0, ids_out_dev, count_out_dev, bitmap_out_dev,
                       scores_out_dev, ws_dev, ws_bytes, stream);
}

int bas_select_topk_weighted(const void* x_dev, int64_t ldx, int batch, int k, int n_keep, int score_kind,
                             const float* chan_scale_dev, const float* block_mult_dev, int32_t* ids_out_dev,
                             int32_t* count_out_dev, uint8_t* bitmap_out_dev, double* scores_out_dev, void* ws_dev,
                             size_t ws_bytes, void* stream) {
  return select_common(x_dev, ldx, batch, k, 0, n_keep, score_kind, 0.0, ids_out_dev, count_out_dev, bitmap_out_dev,
                       scores_out_dev, ws_dev, ws_bytes, stream, chan_scale_dev, block_mult_dev);
}

int bas_select_budget(const void* x_dev, int64_t ldx, int batch, int k, double energy_keep, int min_keep,
                      int32_t* ids_out_dev, int32_t* count_out_dev, uint8_t* bitmap_out_dev, double* scores_out_dev,
                      void* ws_dev, size_t ws_bytes, void* stream) {
  return select_common(x_dev, ldx, batch, k, 1, min_keep, BAS_SCORE_ENERGY, energy_keep, ids_out_dev, count_out_dev,
                       bitmap_out_dev, scores_out_dev, ws_dev, ws_bytes, stream);
}

int bas_select_budget_ex(const void* x_dev, int64_t ldx, int batch, int k, double energy_keep, int min_keep,
                         int score_flags, int32_t* ids_out_dev, int32_t* count_out_dev, uint8_t* bitmap_out_dev,
                         double* scores_out_dev, void* ws_dev, size_t ws_bytes, void* stream) {
  if ((score_flags & ~BAS_SCORE_BF16) != 0) return BAS_ERR_INVALID_ARGUMENT;
  return select_common(x_dev, ldx, batch, k, 1, min_keep, BAS_SCORE_ENERGY | score_flags, energy_keep, ids_out_dev,
                       count_out_dev, bitmap_out_dev, scores_out_dev, ws_dev, ws_bytes, stream);
}

int bas_select_budget_capped(const void* x_dev, int64_t ldx, int batch, int k, double energy_keep, int min_keep,
                             int full_above, int score_flags, int32_t* ids_out_dev, int32_t* count_out_dev,
                             uint8_t* bitmap_out_dev, double* scores_out_dev, void* ws_dev, size_t ws_bytes, void* stream) {
  if ((score_flags & ~BAS_SCORE_BF16) != 0 || full_above < 0) return BAS_ERR_INVALID_ARGUMENT;
  return select_common(x_dev, ldx, batch, k, 1, min_keep, BAS_SCORE_ENERGY | score_flags, energy_keep, ids_out_dev,
                       count_out_dev, bitmap_out_dev, scores_out_dev, ws_dev, ws_bytes, stream, nullptr, nullptr, full_above);
}

int bas_select_gemm(const void* x_dev, int64_t ldx, const void* packed_dev, int batch, int k, int n, int n_keep,
                    int score_kind, double energy_keep, void* y_dev, int64_t ldy, int32_t* ids_out_dev,
                    int32_t* count_out_dev, uint8_t* bitmap_out_dev, double* scores_out_dev, void* gemm_ws_dev,
                    size_t gemm_ws_bytes, void* select_ws_dev, size_t select_ws_bytes, int flags, void* stream) {
  if (ids_out_dev == nullptr || count_out_dev == nullptr || k < kBlockK) return BAS_ERR_INVALID_ARGUMENT;
  const int bf16 = (score_kind & BAS_SCORE_BF16) != 0 ? 1 : 0;
  if (bf16 != ((flags & BAS_GEMM_BF16) != 0 ? 1 : 0)) return BAS_ERR_INVALID_ARGUMENT;   // one dtype for X
  const int kind = score_kind & ~BAS_SCORE_BF16;
  const bool budget = energy_keep >= 0.0;
  const int nb_sel = k / kBlockK;
  if ((kind != BAS_SCORE_NORM && kind != BAS_SCORE_ENERGY) || n_keep < 0 || n_keep > nb_sel ||
      (flags & (3 | BAS_GEMM_IDS_STABLE | BAS_GEMM_X_STABLE | BAS_GEMM_NEXT_INDEPENDENT)) != 0)
    return BAS_ERR_INVALID_ARGUMENT;
  FusedSelect sel;
  sel.mode = budget ? 2 : 1;
  sel.n_keep = n_keep;
  sel.score_kind = budget ? BAS_SCORE_ENERGY : kind;
  sel.nb_sel = nb_sel;
  sel.energy_keep = budget ? energy_keep : 0.0;
  sel.ids_out = ids_out_dev;
  sel.count_out = count_out_dev;
  sel.bitmap_out = bitmap_out_dev;
  sel.scores_out = scores_out_dev;
  // grid sizing: the blocks to expect
  const int k_est = budget ? (nb_sel + 1) / 2 : (n_keep > 0 ? n_keep : 1);
  int st = gemm_impl(nullptr, &sel, x_dev, ldx, packed_dev, nullptr, nullptr, k_est, nullptr, batch, k, n, y_dev, ldy,
                     gemm_ws_dev, gemm_ws_bytes, flags, stream);
  if (st != BAS_ERR_UNSUPPORTED) return st;
  // no cluster for this shape: the two-launch chain, same results
  st = select_common(x_dev, ldx, batch, k, budget ? 1 : 0, n_keep, sel.score_kind | (bf16 ? BAS_SCORE_BF16 : 0),
                     sel.energy_keep, ids_out_dev, count_out_dev, bitmap_out_dev, scores_out_dev, select_ws_dev,
                     select_ws_bytes, stream);
  if (st != BAS_OK) return st;
  return gemm_impl(nullptr, nullptr, x_dev, ldx, packed_dev, ids_out_dev, count_out_dev, budget ? nb_sel : n_keep, nullptr,
                   batch, k, n, y_dev, ldy, gemm_ws_dev, gemm_ws_bytes, flags, stream);
}

// ---------------------------------------------------------------------------------------------
// host-buffer operator
// ---------------------------------------------------------------------------------------------
struct bas_linear {
  int n = 0, k = 0, nb = 0, max_batch = 0;
  cudaStream_t stream = nullptr;
  uint8_t* packed = nullptr;
  __half* x_dev = nullptr;
  __half* y_dev = nullptr;
  // one small device block, mirrored in pinned host memory and fetched with a single copy:
  // [0, 256) the contraction's workspace (status word first), then [nb] ids and [1] count
  void* small_dev = nullptr;
  void* small_pin = nullptr;
  size_t small_bytes = 0;
  int32_t* ids_dev = nullptr;    // inside small_dev
  void* gemm_ws = nullptr;       // inside small_dev
  size_t gemm_ws_bytes = 0;
  void* sel_ws = nullptr;
  size_t sel_ws_bytes = 0;
  void* x_pin = nullptr;         // pinned staging, so that the copies are truly asynchronous
  void* y_pin = nullptr;
  int32_t* ids_pin = nullptr;    // inside small_pin
  long long ldx = 0;
  // the forward in flight (bas_linear_submit_host .. bas_linear_wait)
  bool pending = false, y_direct = false;
  void* pend_y = nullptr;
  int32_t* pend_ids = nullptr;
  int pend_batch = 0, pend_k = 0;
  // recurring forwards, captured as CUDA graphs
  struct FwdGraph {
    int batch, n_keep, score_kind;
    const void* x_src;
    void* y_dst;
    bool want_ids;
    cudaGraphExec_t exec;
    bool failed;
  };
  std::vector<FwdGraph> graphs;
};

static void linear_free(bas_linear* h) {
  if (h == nullptr) return;
  if (h->packed) cudaFree(h->packed);
  if (h->x_dev) cudaFree(h->x_dev);
  if (h->y_dev) cudaFree(h->y_dev);
  if (h->small_dev) cudaFree(h->small_dev);
  if (h->sel_ws) cudaFree(h->sel_ws);
  if (h->x_pin) cudaFreeHost(h->x_pin);
  if (h->y_pin) cudaFreeHost(h->y_pin);
  if (h->small_pin) cudaFreeHost(h->small_pin);
  for (auto& g : h->graphs)
    if (g.exec != nullptr) cudaGraphExecDestroy(g.exec);
  if (h->stream) cudaStreamDestroy(h->stream);
  delete h;
}

int bas_linear_create(bas_linear** out, const void* w_host, int n, int k, int max_batch) {
  if (out == nullptr || w_host == nullptr || n <= 0 || k <= 0 || max_batch <= 0) return BAS_ERR_INVALID_ARGUMENT;
  if (max_batch > BAS_MAX_BATCH) return BAS_ERR_UNSUPPORTED;
  *out = nullptr;
  bas_linear* h = new (std::nothrow) bas_linear();
  if (h == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  h->n = n;
  h->k = k;
  h->nb = (k + kBlockK - 1) / kBlockK;
  h->max_batch = max_batch;
  h->ldx = ((long long)k + 7) / 8 * 8;
  __half* w_dev = nullptr;
  cudaError_t e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
#define BAS_TRY(call)            \
  if (e == cudaSuccess) e = (call)
  BAS_TRY(cudaMalloc(&w_dev, (size_t)n * k * 2));
  BAS_TRY(cudaMalloc(&h->packed, bas_packed_weight_bytes(n, k)));
  BAS_TRY(cudaMalloc(&h->x_dev, (size_t)max_batch * h->ldx * 2));
  BAS_TRY(cudaMalloc(&h->y_dev, (size_t)max_batch * n * 2));
  h->gemm_ws_bytes = bas_gemm_workspace_bytes(max_batch, n);
  h->small_bytes = h->gemm_ws_bytes + sizeof(int32_t) * ((size_t)h->nb + 1);
  BAS_TRY(cudaMalloc(&h->small_dev, h->small_bytes));
  h->gemm_ws = h->small_dev;
  h->ids_dev = (int32_t*)((uint8_t*)h->small_dev + h->gemm_ws_bytes);
  h->sel_ws_bytes = bas_select_workspace_bytes(k);
  BAS_TRY(cudaMalloc(&h->sel_ws, h->sel_ws_bytes));
  BAS_TRY(cudaMallocHost(&h->x_pin, (size_t)max_batch * h->ldx * 2));
  BAS_TRY(cudaMallocHost(&h->y_pin, (size_t)max_batch * n * 2));
  BAS_TRY(cudaMallocHost(&h->small_pin, h->small_bytes));
  h->ids_pin = (int32_t*)((uint8_t*)h->small_pin + h->gemm_ws_bytes);
  BAS_TRY(cudaMemsetAsync(h->x_dev, 0, (size_t)max_batch * h->ldx * 2, h->stream));
  BAS_TRY(cudaMemsetAsync(h->gemm_ws, 0, h->gemm_ws_bytes, h->stream));
  BAS_TRY(cudaMemsetAsync(h->sel_ws, 0, h->sel_ws_bytes, h->stream));
  BAS_TRY(cudaMemcpyAsync(w_dev, w_host, (size_t)n * k * 2, cudaMemcpyHostToDevice, h->stream));
#undef BAS_TRY
  int st = BAS_OK;
  if (e == cudaSuccess) st = bas_pack_weight(w_dev, n, k, k, h->packed, h->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
  if (w_dev) cudaFree(w_dev);
  if (e != cudaSuccess || st != BAS_OK) {
    linear_free(h);
    return e != cudaSuccess ? cuda_fail(e) : st;
  }
  *out = h;
  return BAS_OK;
}

// Host memory that the CUDA driver knows as page-locked (cudaMallocHost / cudaHostRegister) can be
// the source or target of an asynchronous copy itself; anything else goes through the handle's own
// pinned staging buffers.
static bool is_pinned_host(const void* ptr) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeHost;
}

// The stream work of one forward with device-side selection: X host -> device, selection,
// contraction, Y, ids and the status word device -> host.  Nothing is waited for.
static int linear_enqueue_selected(bas_linear* h, const void* x_src, int batch, int n_keep, int score_kind, void* y_dst,
                                   bool want_ids) {
  cudaStream_t s = h->stream;
  const size_t row = (size_t)h->k * 2;
  cudaError_t e = cudaMemcpy2DAsync(h->x_dev, (size_t)h->ldx * 2, x_src, row, row, batch, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return cuda_fail(e);
  int st;
  if (h->ldx == h->k) {
    // selection and contraction: one launch where the shape allows, else two
    st = bas_select_gemm(h->x_dev, h->ldx, h->packed, batch, h->k, h->n, n_keep, score_kind, -1.0, h->y_dev, h->n,
                         h->ids_dev, h->ids_dev + h->nb, nullptr, nullptr, h->gemm_ws, h->gemm_ws_bytes, h->sel_ws,
                         h->sel_ws_bytes, 0, s);
    if (st != BAS_OK) return st;
  } else {
    // K is not a multiple of 8: the selection scores the K real channels, the contraction runs over
    // the zero-padded rows
    st = bas_select_topk(h->x_dev, h->ldx, batch, h->k, n_keep, score_kind, h->ids_dev, h->ids_dev + h->nb, nullptr,
                         nullptr, h->sel_ws, h->sel_ws_bytes, s);
    if (st != BAS_OK) return st;
    st = bas_gemm(h->x_dev, h->ldx, h->packed, h->ids_dev, h->ids_dev + h->nb, n_keep, nullptr, batch, (int)h->ldx, h->n,
                  h->y_dev, h->n, h->gemm_ws, h->gemm_ws_bytes, s);
    if (st != BAS_OK) return st;
  }
  e = cudaMemcpyAsync(y_dst, h->y_dev, (size_t)batch * h->n * 2, cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return cuda_fail(e);
  // status word, and the ids when the caller wants them: one copy
  e = cudaMemcpyAsync(h->small_pin, h->small_dev, want_ids ? h->gemm_ws_bytes + sizeof(int32_t) * n_keep : sizeof(unsigned int),
                      cudaMemcpyDeviceToHost, s);
  return e == cudaSuccess ? BAS_OK : cuda_fail(e);
}

// A forward that recurs with the same sizes and buffers is replayed as one CUDA graph launch instead
// of six stream calls (the host-side cost of a call is mostly those).  The first occurrence runs
// eagerly (it also performs every one-time set-up that must not happen under capture), the second is
// captured, later ones are replays.  BAS_LINEAR_GRAPHS=0 keeps everything eager.
static bool linear_graphs_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("BAS_LINEAR_GRAPHS");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

static int linear_run_selected(bas_linear* h, const void* x_src, int batch, int n_keep, int score_kind, void* y_dst,
                               bool want_ids) {
  if (!linear_graphs_enabled()) return linear_enqueue_selected(h, x_src, batch, n_keep, score_kind, y_dst, want_ids);
  bas_linear::FwdGraph* g = nullptr;
  for (auto& c : h->graphs)
    if (c.batch == batch && c.n_keep == n_keep && c.score_kind == score_kind && c.x_src == x_src && c.y_dst == y_dst &&
        c.want_ids == want_ids)
      g = &c;
  if (g == nullptr) {
    if (h->graphs.size() >= 8) {   // forget the oldest
      if (h->graphs.front().exec != nullptr) cudaGraphExecDestroy(h->graphs.front().exec);
      h->graphs.erase(h->graphs.begin());
    }
    h->graphs.push_back(bas_linear::FwdGraph{batch, n_keep, score_kind, x_src, y_dst, want_ids, nullptr, false});
    return linear_enqueue_selected(h, x_src, batch, n_keep, score_kind, y_dst, want_ids);
  }
  if (g->exec == nullptr && !g->failed) {
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamBeginCapture(h->stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
      const int st = linear_enqueue_selected(h, x_src, batch, n_keep, score_kind, y_dst, want_ids);
      e = cudaStreamEndCapture(h->stream, &graph);
      if (st == BAS_OK && e == cudaSuccess && graph != nullptr) e = cudaGraphInstantiate(&g->exec, graph, 0);
      else if (e == cudaSuccess) e = cudaErrorUnknown;
      if (graph != nullptr) cudaGraphDestroy(graph);
    }
    if (e != cudaSuccess || g->exec == nullptr) {
      (void)cudaGetLastError();
      g->exec = nullptr;
      g->failed = true;
    }
  }
  if (g->exec == nullptr) return linear_enqueue_selected(h, x_src, batch, n_keep, score_kind, y_dst, want_ids);
  const cudaError_t e = cudaGraphLaunch(g->exec, h->stream);
  return e == cudaSuccess ? BAS_OK : cuda_fail(e);
}

// Enqueue one forward on the handle's stream: X host -> device, selection (or the caller's ids),
// contraction, Y (and ids, status word) device -> host.  Nothing is waited for.
static int linear_submit(bas_linear* h, const void* x_host, int batch, int n_keep, int score_kind,
                         const int32_t* ids_host, int n_ids, void* y_host, int32_t* ids_host_out) {
  if (h == nullptr || x_host == nullptr || y_host == nullptr) return BAS_ERR_INVALID_ARGUMENT;
  if (batch <= 0 || batch > h->max_batch) return BAS_ERR_INVALID_ARGUMENT;
  if (h->pending) return BAS_ERR_INVALID_ARGUMENT;   // one forward in flight per handle
  cudaStream_t s = h->stream;
  // host (-> pinned) -> device (rows padded to a multiple of 8 channels; the padding stays zero)
  const size_t row = (size_t)h->k * 2;
  const void* x_src = x_host;
  if (!is_pinned_host(x_host)) {
    std::memcpy(h->x_pin, x_host, row * batch);
    x_src = h->x_pin;
  }
  h->y_direct = is_pinned_host(y_host);
  void* y_dst = h->y_direct ? y_host : h->y_pin;
  int k_host;
  if (ids_host != nullptr || n_ids == 0) {
    if (n_ids < 0 || n_ids > h->nb) return BAS_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaMemcpy2DAsync(h->x_dev, (size_t)h->ldx * 2, x_src, row, row, batch, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return cuda_fail(e);
    if (n_ids > 0) {
      std::memcpy(h->ids_pin, ids_host, sizeof(int32_t) * n_ids);
      e = cudaMemcpyAsync(h->ids_dev, h->ids_pin, sizeof(int32_t) * n_ids, cudaMemcpyHostToDevice, s);
      if (e != cudaSuccess) return cuda_fail(e);
    }
    k_host = n_ids;
    const int st = bas_gemm(h->x_dev, h->ldx, h->packed, h->ids_dev, nullptr, k_host, nullptr, batch, (int)h->ldx, h->n,
                            h->y_dev, h->n, h->gemm_ws, h->gemm_ws_bytes, s);
    if (st != BAS_OK) return st;
    e = cudaMemcpyAsync(y_dst, h->y_dev, (size_t)batch * h->n * 2, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaMemcpyAsync(h->small_pin, h->gemm_ws, sizeof(unsigned int), cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return cuda_fail(e);
    ids_host_out = nullptr;   // the caller's own ids: nothing to hand back
  } else {
    k_host = n_keep;
    const int st = linear_run_selected(h, x_src, batch, n_keep, score_kind, y_dst, ids_host_out != nullptr);
    if (st != BAS_OK) return st;
  }
  h->pending = true;
  h->pend_y = y_host;
  h->pend_ids = ids_host_out;
  h->pend_batch = batch;
  h->pend_k = k_host;
  return BAS_OK;
}

// Wait for the handle's forward in flight and hand its results to the caller's buffers.
static int linear_wait(bas_linear* h) {
  if (h == nullptr || !h->pending) return BAS_ERR_INVALID_ARGUMENT;
  h->pending = false;
  cudaError_t e = cudaStreamSynchronize(h->stream);
  if (e != cudaSuccess) return cuda_fail(e);
  if (!h->y_direct) std::memcpy(h->pend_y, h->y_pin, (size_t)h->pend_batch * h->n * 2);
  if (h->pend_ids != nullptr && h->pend_k > 0) std::memcpy(h->pend_ids, h->ids_pin, sizeof(int32_t) * h->pend_k);
  unsigned int* flag_pin = (unsigned int*)h->small_pin;
  if (*flag_pin != 0) {
    cudaMemsetAsync(h->gemm_ws, 0, sizeof(unsigned int), h->stream);
    return BAS_ERR_DEVICE_FLAG;
  }
  return BAS_OK;
}

static int linear_forward(bas_linear* h, const void* x_host, int batch, int n_keep, int score_kind,
                          const int32_t* ids_host, int n_ids, void* y_host, int32_t* ids_host_out) {
  const int st = linear_submit(h, x_host, batch, n_keep, score_kind, ids_host, n_ids, y_host, ids_host_out);
  return st != BAS_OK ? st : linear_wait(h);
}

int bas_linear_submit_host(bas_linear* h, const void* x_host, int batch, int n_keep, int score_kind, void* y_host,
                           int32_t* ids_host_out) {
  if (h == nullptr || n_keep < 1 || n_keep > h->k / kBlockK) return BAS_ERR_INVALID_ARGUMENT;
  return linear_submit(h, x_host, batch, n_keep, score_kind, nullptr, -1, y_host, ids_host_out);
}

int bas_linear_wait(bas_linear* h) { return linear_wait(h); }

int bas_linear_forward_host(bas_linear* h, const void* x_host, int batch, int n_keep, int score_kind, void* y_host,
                            int32_t* ids_host_out) {
  if (h == nullptr || n_keep < 1 || n_keep > h->k / kBlockK) return BAS_ERR_INVALID_ARGUMENT;
  return linear_forward(h, x_host, batch, n_keep, score_kind, nullptr, -1, y_host, ids_host_out);
}

int bas_linear_forward_host_ids(bas_linear* h, const void* x_host, int batch, const int32_t* ids_host, int n_ids,
                                void* y_host) {
  if (n_ids < 0 || (n_ids > 0 && ids_host == nullptr)) return BAS_ERR_INVALID_ARGUMENT;
  return linear_forward(h, x_host, batch, 0, 0, ids_host, n_ids, y_host, nullptr);
}

void bas_linear_destroy(bas_linear* h) { linear_free(h); }

}  // extern "C"
