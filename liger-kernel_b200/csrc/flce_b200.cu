// Host side of libflce_b200.so: argument checking, workspace carving, TMA tensor maps,
// and kernel launches.
// The exported functions are documented in include/flce_b200.h.
#include "flce_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>
#include <type_traits>

#include "ce_fused_sm100.cuh"
#include "ce_kernels.cuh"
#include "epilogues.cuh"
#include "gemm_sm100.cuh"
#include "head_loss_kernels.cuh"
#include "rmsnorm_rows.cuh"
#include "row_kernels.cuh"

namespace flce {

// ------------------------------------------------------------------ errors
static thread_local char g_last_error[512] = "";

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

#define FLCE_CUDA(expr)                                                                             \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    if (e__ != cudaSuccess) return fail(FLCE_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

// ------------------------------------------------------------------ process-wide options
// (atomics: autograd calls backward from worker threads while another thread may still be setting options)
static std::atomic<long long> g_raster_bytes{32ll << 20};  // bytes of A tiles kept hot per raster group
static std::atomic<int> g_cta_pair{1};           // use CTA pairs (cta_group::2) for the FLCE GEMMs
static std::atomic<int> g_poll_sleep_ns{0};      // epilogue back-off while waiting for an accumulator
static std::atomic<int> g_l2_hints{0};           // 1: mark streamed operands evict-first and re-read ones evict-last
static std::atomic<int> g_n_group{-1};           // n-fastest raster: n-tiles per group (-1 = chosen per GEMM, 0 = all)
static std::atomic<int> g_bulk_store{1};         // store epilogue through TMA stores / adds where it applies
static std::atomic<int> g_ce_store_exp{1};       // one-launch cross-entropy: keep the exponentials of the statistics pass
static std::atomic<int> g_ce_small_slice{kCeFusedSmallSliceBytes};   // slice size the one-launch cross-entropy aims for
static std::atomic<int> g_ce_warps{8};           // warps per CTA of the one-launch cross-entropy: 8 or 16
static std::atomic<int> g_stagger_pct{0};        // wide fp32-accumulating GEMMs: spread of the units' first-tile cut, % of K (0 = off)
static std::atomic<int> g_wide_tiles{1};         // 256 x 512 tiles for the gradient GEMMs of CTA pairs when K is long

// ------------------------------------------------------------------ optional per-kernel timing
// When enabled, every tensor-core launch is bracketed by a pair of CUDA events on the caller's stream;
// flce_b200_profile_read sums the elapsed times per kernel kind.  Off by default (no events, no cost).
enum KernelKind : int { kKindStats = 0, kKindDz = 1, kKindDw = 2, kKindDx = 3, kKindOther = 4, kNumKinds = 5 };
struct ProfileSlot {
  cudaEvent_t start, stop;
  int kind;
};
constexpr int kMaxProfileSlots = 8192;
static bool g_profile_on = false;
static ProfileSlot g_profile[kMaxProfileSlots];
static int g_profile_created = 0;  // events exist for slots [0, created)
static int g_profile_used = 0;
static std::atomic<long long> g_kernel_launches{0};
static std::mutex g_profile_mutex;

static ProfileSlot* profile_begin(int kind, cudaStream_t stream) {
  if (!g_profile_on) return nullptr;
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  if (g_profile_used >= kMaxProfileSlots) return nullptr;
  if (g_profile_used >= g_profile_created) {
    ProfileSlot& fresh = g_profile[g_profile_created];
    if (cudaEventCreate(&fresh.start) != cudaSuccess || cudaEventCreate(&fresh.stop) != cudaSuccess) return nullptr;
    ++g_profile_created;
  }
  ProfileSlot* slot = &g_profile[g_profile_used++];
  slot->kind = kind;
  cudaEventRecord(slot->start, stream);
  return slot;
}
static void profile_end(ProfileSlot* slot, cudaStream_t stream) {
  if (slot != nullptr) cudaEventRecord(slot->stop, stream);
}

// ------------------------------------------------------------------ per-device state
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  int* status = nullptr;  // device word written by abandoned waits
};
static DeviceState g_dev[64];
static std::atomic<int> g_sm_count_hint{0};   // SM count of the first device seen (work-partition heuristics of the planners)
static std::mutex g_dev_mutex;
__device__ int g_device_status_word;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int device_state(DeviceState** out) {
  int dev = 0;
  FLCE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(FLCE_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceState& st = g_dev[dev];
  if (!st.ready) {
    FLCE_CUDA(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
    FLCE_CUDA(cudaDeviceGetAttribute(&st.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    FLCE_CUDA(cudaDeviceGetAttribute(&st.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    if (st.cc_major != 10)
      return fail(FLCE_ERR_UNSUPPORTED, "this library is built for sm_100a only; device %d is sm_%d%d", dev,
                  st.cc_major, st.cc_minor);
    void* p = nullptr;
    FLCE_CUDA(cudaGetSymbolAddress(&p, g_device_status_word));
    st.status = static_cast<int*>(p);
    FLCE_CUDA(cudaMemset(st.status, 0, sizeof(int)));
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      FLCE_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
        return fail(FLCE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    st.ready = true;
    int expected = 0;
    g_sm_count_hint.compare_exchange_strong(expected, st.sm_count);
  }
  *out = &st;
  return FLCE_OK;
}

// 2-D tensor map over a row-major 16-bit matrix: `inner` contiguous elements per row, `outer` rows
// `pitch` elements apart, boxes of box_inner x box_outer, 128-byte swizzle, zero fill outside.
static int make_map(CUtensorMap* map, const void* base, int dtype, long long inner, long long outer, long long pitch,
                    int box_inner, int box_outer) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "matrix base %p is not 16-byte aligned", base);
  if ((pitch * 2) % 16 != 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "row pitch %lld elements is not a multiple of 8", pitch);
  if (inner <= 0 || outer <= 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "empty matrix (%lld x %lld)", outer, inner);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = (dtype == FLCE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FLCE_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return FLCE_OK;
}

// 2-D tensor map for TMA stores of 32 x 32 patches of a row-major output (fp32: 128-byte swizzle in shared memory;
// 16-bit: dense 64-byte rows).  `fmt` is an OutFormat.
static int make_store_map(CUtensorMap* map, void* base, int fmt, long long cols, long long rows, long long pitch) {
  const int esize = fmt == kOutFp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch * esize) % 16 != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "output base %p / pitch %lld elements is not 16-byte aligned", base, pitch);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch) * esize};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = fmt == kOutFp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : (fmt == kOutBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r = g_encode(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        fmt == kOutFp32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FLCE_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", static_cast<int>(r));
  return FLCE_OK;
}

// An operand of D = A.B^T as the main loop wants it.
struct Operand {
  const void* base;
  long long rows;   // extent along M (for A) or N (for B)
  long long depth;  // extent along K
  long long pitch;  // elements between consecutive rows of the *stored* matrix
  int mn_major;     // 0: stored [rows][depth]; 1: stored [depth][rows]
};

static int operand_map(CUtensorMap* map, const Operand& op, int dtype, int tile_rows) {
  if (op.mn_major == 0) return make_map(map, op.base, dtype, op.depth, op.rows, op.pitch, kBlockK, tile_rows);
  return make_map(map, op.base, dtype, op.rows, op.depth, op.pitch, 64, kBlockK);
}

static long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// n-tiles per raster group of an n-fastest GEMM, chosen by estimated DRAM traffic.  A group walks all m-tiles over g n-tiles, so
// the g B panels (tile_n x K each) are what is re-read.  While they fit a third of L2 they stay resident and every A panel is
// read once per group; otherwise a wave of `units` tiles touches units / g A panels and g B panels, and nothing survives to
// the next wave.  Smaller groups re-read A more often, larger ones re-read B: the estimate picks between the halvings of n_tiles.
static int raster_n_group_for(int m_tiles, int n_tiles, long long K, int tile_m, int tile_n, int units) {
  const double a_panel = 2.0 * tile_m * K, b_panel = 2.0 * tile_n * K;
  const double resident = 40.0 * 1024 * 1024;
  const double waves = static_cast<double>(m_tiles) * n_tiles / (units > 0 ? units : 1);
  int best = n_tiles;
  double best_bytes = -1.0;
  for (int g = n_tiles; g >= 1; g = (g + 1) / 2) {
    double bytes;
    if (g * b_panel <= resident)
      bytes = a_panel * m_tiles * ((n_tiles + g - 1) / g) + b_panel * n_tiles;
    else
      bytes = (a_panel * (static_cast<double>(units) / g < m_tiles ? static_cast<double>(units) / g : m_tiles) + b_panel * g) *
              (waves < 1.0 ? 1.0 : waves);
    if (best_bytes < 0 || bytes < best_bytes * 0.97) {   // a smaller group has to win by 3 % to be taken
      best_bytes = bytes;
      best = g;
    }
    if (g == 1) break;
  }
  return best;
}

template <int kCtas, int kAMajor, int kBMajor, class Epi, int kNSub = 1>
static int launch_gemm_impl(const DeviceState& dev, int kind, const Operand& a, const Operand& b, int dtype, long long M,
                            long long N, long long K, long long raster_row_bytes, bool n_fastest,
                            const typename Epi::Params& ep, cudaStream_t stream, const int* active_rows, int active_role,
                            int active_base, const int* gate, int reserve_sms) {
  using Cfg = StageCfg<kCtas, kNSub>;
  CUtensorMap map_a, map_b, map_d;
  int rc = operand_map(&map_a, a, dtype, kBlockM);
  if (rc != FLCE_OK) return rc;
  rc = operand_map(&map_b, b, dtype, kBlockN / kCtas);
  if (rc != FLCE_OK) return rc;
  map_d = map_a;   // unused unless the epilogue stores through TMA
  typename Epi::Params ep_launch = ep;
  if constexpr (std::is_same<Epi, StoreEpilogue>::value) {
    // one destination, nothing read back: the patches leave as TMA stores / adds
    const bool one_dst = (ep.out != nullptr) != (ep.acc_out != nullptr);
    ep_launch.bulk = (g_bulk_store.load() != 0 && ep.acc_in == nullptr && one_dst) ? 1 : 0;
    if (ep_launch.bulk) {
      if (ep.acc_out != nullptr) rc = make_store_map(&map_d, ep.acc_out, kOutFp32, ep.n_cols, ep.m_rows, ep.ld_acc);
      else rc = make_store_map(&map_d, ep.out, ep.out_fmt, ep.n_cols, ep.m_rows, ep.ld_out);
      if (rc != FLCE_OK) return rc;
    }
  }
  GemmShape shape;
  shape.M = static_cast<int>(M);
  shape.N = static_cast<int>(N);
  shape.K = static_cast<int>(K);
  shape.m_tiles = static_cast<int>(ceil_div(M, kBlockM * kCtas));
  shape.n_tiles = static_cast<int>(ceil_div(N, kBlockN * kNSub));
  shape.k_blocks = static_cast<int>(ceil_div(K, kBlockK));
  shape.poll_sleep_ns = g_poll_sleep_ns;
  shape.active_rows = active_rows;
  shape.active_role = active_rows != nullptr ? active_role : 0;
  shape.active_base = active_base;
  shape.gate = gate;
  shape.stagger = 0;
  if constexpr (std::is_same<Epi, StoreEpilogue>::value && kNSub == 2) {
    // fp32 accumulator output, nothing read back: the first tile of every unit may be cut in two (tile_schedule.cuh)
    if (ep.acc_out != nullptr && ep.acc_in == nullptr && ep.out == nullptr) shape.stagger = g_stagger_pct.load();
  }
  shape.hint_a = 0;
  shape.hint_b = 0;
  if (g_l2_hints) {
    // sweeps over the vocabulary re-read X tiles (A) and stream W (B); the gradient GEMMs stream dZ (A) and re-read B
    shape.hint_a = n_fastest ? 1 : 2;
    shape.hint_b = n_fastest ? 2 : 1;
  }
  if (n_fastest) {
    shape.group_along_m = 0;
    int n_group = g_n_group.load();
    if (n_group < 0) n_group = raster_n_group_for(shape.m_tiles, shape.n_tiles, K, kBlockM * kCtas, kBlockN * kNSub,
                                                   dev.sm_count / kCtas);
    shape.group = (n_group > 0 && n_group < shape.n_tiles) ? n_group : shape.n_tiles;
  } else {
    shape.group_along_m = 1;
    long long g = g_raster_bytes.load() / (raster_row_bytes > 0 ? raster_row_bytes : 1);
    if (g < 1) g = 1;
    if (g > shape.m_tiles) g = shape.m_tiles;
    shape.group = static_cast<int>(g);
  }
  const long long tiles = static_cast<long long>(shape.m_tiles) * shape.n_tiles;
  // reserve_sms: SMs left free for a kernel of the caller's that should run beside this one (a collective)
  long long units = (dev.sm_count - reserve_sms) / kCtas;
  if (units < 1) units = 1;
  if (units > tiles) units = tiles;
  auto kernel = gemm_tcgen05_kernel<kCtas, kAMajor, kBMajor, Epi, kNSub>;
  {  // once per instantiation and device
    static std::atomic<bool> smem_set[64];
    int ordinal = 0;
    FLCE_CUDA(cudaGetDevice(&ordinal));
    if (!smem_set[ordinal & 63].load(std::memory_order_acquire)) {
      FLCE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
      smem_set[ordinal & 63].store(true, std::memory_order_release);
    }
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(units * kCtas), 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = kCtas;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  const int fmt = (dtype == FLCE_BF16) ? 1 : 0;
  ProfileSlot* slot = profile_begin(kind, stream);
  const cudaError_t launched = cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_d, shape, fmt, ep_launch, dev.status);
  profile_end(slot, stream);
  if (launched != cudaSuccess) return fail(FLCE_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(launched));
  ++g_kernel_launches;
  return FLCE_OK;
}

template <int kAMajor, int kBMajor, class Epi>
static int launch_gemm(const DeviceState& dev, int kind, bool pair, const Operand& a, const Operand& b, int dtype, long long M,
                       long long N, long long K, long long raster_row_bytes, bool n_fastest,
                       const typename Epi::Params& ep, cudaStream_t stream, const int* active_rows = nullptr,
                       int active_role = 0, int active_base = 0, const int* gate = nullptr, int reserve_sms = 0) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "empty GEMM %lld x %lld x %lld", M, N, K);
  if (M > 0x7fffffffll || N > 0x7fffffffll || K > 0x7fffffffll)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "GEMM extent does not fit 32 bits");
  if constexpr (std::is_same<Epi, StoreEpilogue>::value) {
    // long K, light epilogue, enough columns to fill 512-wide tiles: the wide form moves a quarter less data per product
    if (pair && g_wide_tiles && K >= 2048 && N >= 1024)
      return launch_gemm_impl<2, kAMajor, kBMajor, Epi, 2>(dev, kind, a, b, dtype, M, N, K, raster_row_bytes * 2, n_fastest, ep,
                                                           stream, active_rows, active_role, active_base, gate, reserve_sms);
  }
  if (pair)
    return launch_gemm_impl<2, kAMajor, kBMajor, Epi>(dev, kind, a, b, dtype, M, N, K, raster_row_bytes * 2, n_fastest, ep, stream,
                                                      active_rows, active_role, active_base, gate, reserve_sms);
  return launch_gemm_impl<1, kAMajor, kBMajor, Epi>(dev, kind, a, b, dtype, M, N, K, raster_row_bytes, n_fastest, ep, stream,
                                                    active_rows, active_role, active_base, gate, reserve_sms);
}

// (the small SIMT kernels live in row_kernels.cuh)

// ------------------------------------------------------------------ problem checks / workspace plans
static int check_problem(const flce_problem_t* p) {
  if (p == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "problem is NULL");
  if (p->n_rows <= 0 || p->hidden <= 0 || p->vocab <= 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "shapes must be positive (n_rows=%lld hidden=%lld vocab=%lld)",
                (long long)p->n_rows, (long long)p->hidden, (long long)p->vocab);
  if (p->n_rows > 0x7fffffffll || p->vocab > 0x7fffffffll || p->hidden > 0x7fffffffll)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "shapes must fit 32 bits");
  if (p->dtype != FLCE_BF16 && p->dtype != FLCE_FP16)
    return fail(FLCE_ERR_UNSUPPORTED, "x / w must be bf16 or fp16 (dtype code %d)", p->dtype);
  if (p->hidden % 8 != 0 || p->ld_x % 8 != 0 || p->ld_w % 8 != 0 || p->ld_x < p->hidden || p->ld_w < p->hidden)
    return fail(FLCE_ERR_INVALID_ARGUMENT,
                "hidden (%lld) and row pitches (%lld, %lld) must be multiples of 8 elements (16-byte rows)",
                (long long)p->hidden, (long long)p->ld_x, (long long)p->ld_w);
  if (p->x == nullptr || p->w == nullptr || p->target == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "x, w and target must not be NULL");
  if (p->reduction < FLCE_MEAN || p->reduction > FLCE_NONE) return fail(FLCE_ERR_INVALID_ARGUMENT, "bad reduction");
  if (!(p->label_smoothing >= 0.f && p->label_smoothing <= 1.f))
    return fail(FLCE_ERR_INVALID_ARGUMENT, "label_smoothing must be in [0, 1]");
  if (p->softcap < 0.f) return fail(FLCE_ERR_INVALID_ARGUMENT, "softcap must be positive (0 = off)");
  if (p->vocab_total < p->vocab || p->vocab_offset < 0 || p->vocab_offset + p->vocab > p->vocab_total)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "vocabulary shard [%lld, %lld) does not fit vocab_total %lld",
                (long long)p->vocab_offset, (long long)(p->vocab_offset + p->vocab), (long long)p->vocab_total);
  if (p->ce_weight != nullptr && p->vocab != p->vocab_total)
    return fail(FLCE_ERR_UNSUPPORTED, "class weights are not supported together with vocabulary sharding");
  return FLCE_OK;
}

static RowMath row_math(const flce_problem_t* p) {
  RowMath rm;
  rm.ignore_index = p->ignore_index;
  rm.alpha = p->label_smoothing;
  rm.eps = p->label_smoothing / static_cast<float>(p->vocab_total);
  rm.lambda = p->lse_square_scale;
  rm.mean = p->reduction == FLCE_MEAN;
  rm.token_scaling = p->use_token_scaling != 0;
  rm.weighted = p->ce_weight != nullptr;
  rm.vocab = p->vocab;
  rm.vocab_offset = p->vocab_offset;
  return rm;
}

struct ForwardPlan {
  int n_tiles;
  size_t plane;  // bytes of one [n_tiles][n_rows] fp32 plane
  size_t total;
};
static ForwardPlan forward_plan(const flce_problem_t* p) {
  ForwardPlan f;
  f.n_tiles = static_cast<int>(ceil_div(p->vocab, kBlockN));
  f.plane = align_up(static_cast<size_t>(f.n_tiles) * p->n_rows * sizeof(float), 256);
  f.total = 5 * f.plane;
  return f;
}

struct BackwardPlan {
  long long slab_cols;  // vocabulary columns per slab
  long long ld_dz;
  int n_slabs;
  size_t coef_bytes, slab_bytes, acc_bytes, total;
};
static BackwardPlan backward_plan(const flce_problem_t* p, size_t budget, bool need_acc) {
  BackwardPlan b;
  if (budget == 0) budget = size_t(1) << 30;
  long long max_cols = static_cast<long long>(budget / (static_cast<size_t>(p->n_rows) * 2));
  max_cols = max_cols / kBlockN * kBlockN;
  if (max_cols < kBlockN) max_cols = kBlockN;
  b.n_slabs = static_cast<int>(ceil_div(p->vocab, max_cols));
  b.slab_cols = ceil_div(ceil_div(p->vocab, b.n_slabs), kBlockN) * kBlockN;
  b.n_slabs = static_cast<int>(ceil_div(p->vocab, b.slab_cols));
  b.ld_dz = b.slab_cols;
  b.coef_bytes = align_up(static_cast<size_t>(p->n_rows) * 3 * sizeof(float), 256);
  b.slab_bytes = align_up(static_cast<size_t>(p->n_rows) * b.ld_dz * 2, 256);
  b.acc_bytes = (need_acc && b.n_slabs > 1) ? align_up(static_cast<size_t>(p->n_rows) * p->hidden * sizeof(float), 256) : 0;
  b.total = b.coef_bytes + b.slab_bytes + b.acc_bytes;
  return b;
}

// single-sweep mode: token chunks with the chunk's soft-capped logits kept in a 16-bit slab [chunk][ld]
struct FusedPlan {
  long long chunk_rows, ld_slab;
  int n_chunks, n_tiles;
  size_t plane, rowstats_bytes, coef_bytes, slab_bytes, acc_bytes, total;
  // exp-store form: per-row reference points (all rows), per-chunk alpha and scaled copy of x, label-smoothing vectors
  size_t shift_bytes, alpha_bytes, xs_bytes, vec_bytes, colsum_scratch_bytes, flag_bytes, exp_bytes;
};
static FusedPlan fused_plan(const flce_problem_t* p, size_t budget, bool need_acc) {
  FusedPlan f;
  if (budget == 0) budget = size_t(5) << 29;  // 2.5 GiB
  f.ld_slab = ceil_div(p->vocab, 64) * 64;
  long long max_rows = static_cast<long long>(budget / (static_cast<size_t>(f.ld_slab) * 2));
  max_rows = max_rows / 256 * 256;
  if (max_rows < 256) max_rows = 256;
  if (max_rows > 65280) max_rows = 65280;  // the in-place gradient kernel puts the chunk's rows on grid.y
  f.n_chunks = static_cast<int>(ceil_div(p->n_rows, max_rows));
  f.chunk_rows = ceil_div(ceil_div(p->n_rows, f.n_chunks), 256) * 256;
  if (f.n_chunks > 1) {
    // The grad_input GEMM of a chunk has few, long tiles (K = vocabulary): (chunk rows / 256) x ceil(hidden / 512) of them on
    // 74 CTA pairs.  Pick the chunk height, within 3/4 .. 1 of what the budget allows, that needs the fewest waves of such
    // tiles over the whole problem (equal chunks of 8192 rows at the Llama-3-8B head: 4 x 4 waves with the last one 46 % full;
    // chunks of 9472: 3 x 4 full waves + 2); ties go to the taller chunk.
    const int sms = g_sm_count_hint.load();
    const long long units = (sms > 1 ? sms : 148) / 2;
    const long long n_wide = ceil_div(p->hidden, 2 * kBlockN);
    long long best_rows = f.chunk_rows, best_waves = -1;
    for (long long rows = max_rows; rows >= 256 && rows * 4 >= max_rows * 3; rows -= 256) {
      long long waves = 0;
      for (long long r0 = 0; r0 < p->n_rows; r0 += rows) {
        const long long here = (p->n_rows - r0 < rows) ? p->n_rows - r0 : rows;
        waves += ceil_div(ceil_div(here, 256) * n_wide, units);
      }
      if (best_waves < 0 || waves < best_waves) {
        best_waves = waves;
        best_rows = rows;
      }
    }
    f.chunk_rows = best_rows;
  }
  f.n_chunks = static_cast<int>(ceil_div(p->n_rows, f.chunk_rows));
  f.n_tiles = static_cast<int>(ceil_div(p->vocab, kBlockN));
  f.plane = align_up(static_cast<size_t>(f.n_tiles) * f.chunk_rows * sizeof(float), 256);
  f.rowstats_bytes = align_up(static_cast<size_t>(FLCE_ROWSTAT_PLANES) * f.chunk_rows * sizeof(float), 256);
  f.coef_bytes = align_up(static_cast<size_t>(f.chunk_rows) * 3 * sizeof(float), 256);
  f.slab_bytes = align_up(static_cast<size_t>(f.chunk_rows) * f.ld_slab * 2, 256);
  f.acc_bytes = (need_acc && f.n_chunks > 1) ? align_up(static_cast<size_t>(p->vocab) * p->hidden * sizeof(float), 256) : 0;
  f.shift_bytes = align_up(static_cast<size_t>(p->n_rows) * sizeof(float), 256);
  f.alpha_bytes = align_up(static_cast<size_t>(f.chunk_rows) * sizeof(float), 256);
  f.xs_bytes = align_up(static_cast<size_t>(f.chunk_rows) * p->hidden * 2, 256);
  f.vec_bytes = align_up(static_cast<size_t>(p->hidden) * sizeof(float), 256);          // one of: sum_j w_j W_j, sum_r c2_r x_r
  f.colsum_scratch_bytes = align_up(static_cast<size_t>(kColsumSplits) * p->hidden * sizeof(float), 256);
  f.flag_bytes = align_up(static_cast<size_t>(f.n_chunks) * sizeof(int), 256);
  f.exp_bytes = f.shift_bytes + f.alpha_bytes + f.xs_bytes + 2 * f.vec_bytes + f.colsum_scratch_bytes + f.flag_bytes;
  f.total = 5 * f.plane + f.rowstats_bytes + f.coef_bytes + f.slab_bytes + f.exp_bytes + f.acc_bytes;
  return f;
}

// ------------------------------------------------------------------ stand-alone cross-entropy
static int check_ce_problem(const flce_ce_problem_t* p) {
  if (p == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "problem is NULL");
  if (p->n_rows <= 0 || p->vocab <= 0 || p->ld < p->vocab)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "bad logits shape (n_rows=%lld vocab=%lld ld=%lld)", (long long)p->n_rows,
                (long long)p->vocab, (long long)p->ld);
  if (p->n_rows > 0x7fffffffll || p->vocab > 0x7fffffffll) return fail(FLCE_ERR_INVALID_ARGUMENT, "shapes must fit 32 bits");
  if (p->dtype < FLCE_BF16 || p->dtype > FLCE_FP32) return fail(FLCE_ERR_UNSUPPORTED, "logits must be bf16, fp16 or fp32");
  if (p->logits == nullptr || p->target == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "logits and target must not be NULL");
  if (p->reduction < FLCE_MEAN || p->reduction > FLCE_NONE) return fail(FLCE_ERR_INVALID_ARGUMENT, "bad reduction");
  if (!(p->label_smoothing >= 0.f && p->label_smoothing <= 1.f))
    return fail(FLCE_ERR_INVALID_ARGUMENT, "label_smoothing must be in [0, 1]");
  if (p->softcap < 0.f) return fail(FLCE_ERR_INVALID_ARGUMENT, "softcap must be positive (0 = off)");
  return FLCE_OK;
}

static RowMath ce_row_math(const flce_ce_problem_t* p) {
  RowMath rm;
  rm.ignore_index = p->ignore_index;
  rm.alpha = p->label_smoothing;
  rm.eps = p->label_smoothing / static_cast<float>(p->vocab);
  rm.lambda = p->lse_square_scale;
  rm.mean = p->reduction == FLCE_MEAN;
  rm.token_scaling = 0;
  rm.weighted = p->ce_weight != nullptr;
  rm.vocab = p->vocab;
  rm.vocab_offset = 0;
  return rm;
}

static bool ce_rows_vectorisable(const void* base, long long ld, int dtype) {
  const long long esize = dtype == FLCE_FP32 ? 4 : 2;
  return (reinterpret_cast<uintptr_t>(base) & 15) == 0 && (ld * esize) % 16 == 0;
}

template <typename T>
static void launch_ce_stats(const flce_ce_problem_t* p, float* rowstats, cudaStream_t stream) {
  const float inv = p->softcap > 0.f ? 1.f / p->softcap : 0.f;
  const T* x = static_cast<const T*>(p->logits);
  const long long* tgt = reinterpret_cast<const long long*>(p->target);
  const unsigned grid = static_cast<unsigned>(p->n_rows);
  if (ce_rows_vectorisable(p->logits, p->ld, p->dtype))
    ce_stats_kernel<T, true><<<grid, kCeThreads, 0, stream>>>(x, p->ld, static_cast<int>(p->n_rows), static_cast<int>(p->vocab),
                                                             tgt, p->ce_weight, p->softcap, inv, rowstats);
  else
    ce_stats_kernel<T, false><<<grid, kCeThreads, 0, stream>>>(x, p->ld, static_cast<int>(p->n_rows), static_cast<int>(p->vocab),
                                                              tgt, p->ce_weight, p->softcap, inv, rowstats);
}

template <typename T>
static void launch_ce_grad(const flce_ce_problem_t* p, void* grad, long long ld_grad, const float* lse, const float* c1,
                           const float* c2, const float* c3, cudaStream_t stream) {
  const float inv = p->softcap > 0.f ? 1.f / p->softcap : 0.f;
  const T* x = static_cast<const T*>(p->logits);
  const long long* tgt = reinterpret_cast<const long long*>(p->target);
  const bool vec = ce_rows_vectorisable(p->logits, p->ld, p->dtype) && ce_rows_vectorisable(grad, ld_grad, p->dtype);
  const long long per_thread = vec ? CeElem<T>::kVec : 1;
  dim3 grid(static_cast<unsigned>(p->n_rows),
            static_cast<unsigned>(ceil_div(ceil_div(p->vocab, per_thread), kCeThreads * kCeGradUnroll)), 1);
  if (vec)
    ce_grad_kernel<T, true><<<grid, kCeThreads, 0, stream>>>(x, p->ld, static_cast<T*>(grad), ld_grad, static_cast<int>(p->n_rows),
                                                            static_cast<int>(p->vocab), tgt, p->ce_weight, p->softcap, inv, lse,
                                                            c1, c2, c3);
  else
    ce_grad_kernel<T, false><<<grid, kCeThreads, 0, stream>>>(x, p->ld, static_cast<T*>(grad), ld_grad,
                                                             static_cast<int>(p->n_rows), static_cast<int>(p->vocab), tgt,
                                                             p->ce_weight, p->softcap, inv, lse, c1, c2, c3);
}

// Cluster size and slice (in 16-byte vectors) of ce_fused_kernel for a row of `vocab` elements, or false when the row does not
// qualify: prefers slices small enough for three CTAs per SM, then one CTA per SM, over at most eight CTAs.
static bool ce_fused_geometry(long long vocab, long long esize, int* cluster, int* slice_vecs) {
  const long long per_vec = 16 / esize;
  if (vocab % per_vec != 0) return false;
  const long long n_vec = vocab / per_vec;
  for (const long long limit : {static_cast<long long>(g_ce_small_slice.load()), static_cast<long long>(kCeFusedMaxSliceBytes)})
    for (int c = 1; c <= kCeFusedMaxCluster; c *= 2) {
      const long long sv = ceil_div(n_vec, c);
      if (sv * 16 <= limit) {
        *cluster = c;
        *slice_vecs = static_cast<int>(sv);
        return true;
      }
    }
  return false;
}

template <typename T, bool kStoreExp, int kWarps>
static int launch_ce_fused(const flce_ce_problem_t* p, void* grad, long long ld_grad, const float* norm, const CeFusedOut& out,
                           int cluster, int slice_vecs, const DeviceState& dev, cudaStream_t stream) {
  auto* kernel = ce_fused_kernel<T, kStoreExp, kWarps>;
  {  // once per instantiation and device
    static std::atomic<bool> smem_set[64];
    int ordinal = 0;
    FLCE_CUDA(cudaGetDevice(&ordinal));
    if (!smem_set[ordinal & 63].load(std::memory_order_acquire)) {
      FLCE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCeFusedMaxSliceBytes));
      smem_set[ordinal & 63].store(true, std::memory_order_release);
    }
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(p->n_rows * cluster), 1, 1);
  cfg.blockDim = dim3(kWarps * 32, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(slice_vecs) * 16;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float inv = p->softcap > 0.f ? 1.f / p->softcap : 0.f;
  FLCE_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<const T*>(p->logits), static_cast<long long>(p->ld), static_cast<T*>(grad),
                               ld_grad, static_cast<int>(p->n_rows), static_cast<int>(p->vocab), slice_vecs,
                               reinterpret_cast<const long long*>(p->target), p->ce_weight, p->softcap, inv, ce_row_math(p), norm,
                               out, dev.status));
  return FLCE_OK;
}

// ---- launchers of the chunked sibling losses' row kernels (head_loss_kernels.cuh)
template <typename T>
static void launch_scaled_ce_rows(const void* logits, int64_t ld, int32_t dtype, int64_t n_rows, int64_t vocab,
                                  const long long* target, long long ignore_index, float inv_t, float* nll, float* entropy,
                                  float* lse, cudaStream_t stream) {
  const T* x = static_cast<const T*>(logits);
  const unsigned grid = static_cast<unsigned>(n_rows);
  if (ce_rows_vectorisable(logits, ld, dtype))
    scaled_ce_rows_kernel<T, true><<<grid, kCeThreads, 0, stream>>>(x, ld, static_cast<int>(n_rows), static_cast<int>(vocab),
                                                                   target, ignore_index, inv_t, nll, entropy, lse);
  else
    scaled_ce_rows_kernel<T, false><<<grid, kCeThreads, 0, stream>>>(x, ld, static_cast<int>(n_rows), static_cast<int>(vocab),
                                                                    target, ignore_index, inv_t, nll, entropy, lse);
}

template <typename T>
static void launch_scaled_ce_grad(void* logits, int64_t ld, int32_t dtype, int64_t n_rows, int64_t vocab, const long long* target,
                                  long long ignore_index, float inv_t, const float* lse, const float* entropy,
                                  const float* grad_nll, const float* grad_entropy, cudaStream_t stream) {
  const bool vec = ce_rows_vectorisable(logits, ld, dtype);
  const long long per_thread = vec ? CeElem<T>::kVec : 1;
  dim3 grid(static_cast<unsigned>(n_rows), static_cast<unsigned>(ceil_div(ceil_div(vocab, per_thread), kCeThreads)), 1);
  T* x = static_cast<T*>(logits);
  if (vec)
    scaled_ce_grad_kernel<T, true><<<grid, kCeThreads, 0, stream>>>(x, ld, static_cast<int>(n_rows), static_cast<int>(vocab), target,
                                                                   ignore_index, inv_t, lse, entropy, grad_nll, grad_entropy);
  else
    scaled_ce_grad_kernel<T, false><<<grid, kCeThreads, 0, stream>>>(x, ld, static_cast<int>(n_rows), static_cast<int>(vocab), target,
                                                                    ignore_index, inv_t, lse, entropy, grad_nll, grad_entropy);
}

template <typename T>
static void launch_jsd_rows(int sm_count, void* student, int64_t ld_s, const void* teacher, int64_t ld_t, int32_t dtype,
                            int64_t n_rows, int64_t vocab, const long long* labels, long long ignore_index, float beta, float inv_t,
                            const float* count, float fixed_count, float* loss_rows, cudaStream_t stream) {
  const bool vec = ce_rows_vectorisable(student, ld_s, dtype) && ce_rows_vectorisable(teacher, ld_t, dtype);
  const unsigned grid = static_cast<unsigned>(n_rows < sm_count ? n_rows : sm_count);   // one CTA per SM walks over the rows
  T* xs = static_cast<T*>(student);
  const T* xt = static_cast<const T*>(teacher);
  if (vec)
    jsd_rows_kernel<T, true><<<grid, kJsdThreads, 0, stream>>>(xs, ld_s, xt, ld_t, static_cast<int>(n_rows), static_cast<int>(vocab),
                                                             labels, ignore_index, beta, inv_t, count, fixed_count, loss_rows);
  else
    jsd_rows_kernel<T, false><<<grid, kJsdThreads, 0, stream>>>(xs, ld_s, xt, ld_t, static_cast<int>(n_rows), static_cast<int>(vocab),
                                                              labels, ignore_index, beta, inv_t, count, fixed_count, loss_rows);
}

// ---- the final RMSNorm folded into the two row moves (rmsnorm_rows.cuh)
static int check_rmsnorm(int32_t dtype, int64_t hidden, int32_t casting_mode, const void* gamma) {
  if (dtype != FLCE_BF16 && dtype != FLCE_FP16) return fail(FLCE_ERR_UNSUPPORTED, "the fused RMSNorm takes bf16 or fp16 hidden states");
  if (hidden <= 0 || hidden % 8 != 0) return fail(FLCE_ERR_UNSUPPORTED, "the fused RMSNorm needs a hidden size that is a multiple of 8");
  if (hidden > 512ll * kRmsMaxVecs * 8) return fail(FLCE_ERR_UNSUPPORTED, "the fused RMSNorm handles hidden sizes up to 16384");
  if (casting_mode != kRmsModeLlama && casting_mode != kRmsModeGemma)
    return fail(FLCE_ERR_UNSUPPORTED, "casting_mode must be 0 (llama) or 1 (gemma)");
  if (gamma == nullptr || (reinterpret_cast<uintptr_t>(gamma) & 15) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "the norm weight must be given and 16-byte aligned");
  return FLCE_OK;
}

static int rmsnorm_partial_blocks() {
  int sms = g_sm_count_hint.load();
  if (sms <= 0) sms = 148;
  return 2 * sms;
}

template <typename T>
static void launch_rmsnorm_backward(const void* gy, long long ld_g, const void* x, long long ld_x, const void* gamma,
                                    const float* rstd, const int* perm, const int* active, long long n_rows, long long hidden,
                                    float offset, int mode, void* gx, long long ld_gx, float* partials, int blocks,
                                    cudaStream_t stream) {
  const long long n_vec = hidden / 8;
  const int threads = n_vec <= 256 * kRmsMaxVecs ? 256 : 512;
  const long long per_thread = ceil_div(n_vec, threads);
  auto go = [&](auto kernel) {
    kernel<<<blocks, threads, 0, stream>>>(static_cast<const T*>(gy), ld_g, static_cast<const T*>(x), ld_x,
                                          static_cast<const T*>(gamma), rstd, perm, active, static_cast<int>(n_rows),
                                          static_cast<int>(hidden), offset, mode, static_cast<T*>(gx), ld_gx, partials);
  };
  if (per_thread <= 1) go(rmsnorm_backward_scatter_kernel<T, 1>);
  else if (per_thread <= 2) go(rmsnorm_backward_scatter_kernel<T, 2>);
  else go(rmsnorm_backward_scatter_kernel<T, 4>);
}

}  // namespace flce

using namespace flce;

// ====================================================================================== C ABI
extern "C" {

const char* flce_b200_last_error(void) { return g_last_error; }
const char* flce_b200_version(void) { return "flce_b200 0.1 (sm_100a, tcgen05/TMA)"; }

const char* flce_b200_status_string(int status) {
  switch (status) {
    case FLCE_OK: return "ok";
    case FLCE_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FLCE_ERR_UNSUPPORTED: return "unsupported";
    case FLCE_ERR_WORKSPACE: return "workspace too small";
    case FLCE_ERR_CUDA: return "CUDA error";
    case FLCE_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

int flce_b200_set_option(const char* name, int64_t value) {
  if (name == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "option name is NULL");
  if (strcmp(name, "raster_group_bytes") == 0) {
    if (value <= 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "raster_group_bytes must be positive");
    g_raster_bytes = value;
    return FLCE_OK;
  }
  if (strcmp(name, "cta_pair") == 0) {
    g_cta_pair = value != 0;
    return FLCE_OK;
  }
  if (strcmp(name, "poll_sleep_ns") == 0) {
    if (value < 0 || value > 100000) return fail(FLCE_ERR_INVALID_ARGUMENT, "poll_sleep_ns out of range");
    g_poll_sleep_ns = static_cast<int>(value);
    return FLCE_OK;
  }
  if (strcmp(name, "l2_hints") == 0) {
    g_l2_hints = value != 0;
    return FLCE_OK;
  }
  if (strcmp(name, "bulk_store") == 0) {
    g_bulk_store = value != 0;
    return FLCE_OK;
  }
  if (strcmp(name, "wide_tiles") == 0) {
    g_wide_tiles = value != 0;
    return FLCE_OK;
  }
  if (strcmp(name, "stagger_pct") == 0) {
    if (value < 0 || value > 100) return fail(FLCE_ERR_INVALID_ARGUMENT, "stagger_pct must be 0 .. 100");
    g_stagger_pct = static_cast<int>(value);
    return FLCE_OK;
  }
  if (strcmp(name, "ce_store_exp") == 0) {
    g_ce_store_exp = value != 0;
    return FLCE_OK;
  }
  if (strcmp(name, "ce_warps") == 0) {
    if (value != 8 && value != 16) return fail(FLCE_ERR_INVALID_ARGUMENT, "ce_warps must be 8 or 16");
    g_ce_warps = static_cast<int>(value);
    return FLCE_OK;
  }
  if (strcmp(name, "ce_slice_bytes") == 0) {
    if (value < 16 || value > kCeFusedMaxSliceBytes) return fail(FLCE_ERR_INVALID_ARGUMENT, "ce_slice_bytes out of range");
    g_ce_small_slice = static_cast<int>(value);
    return FLCE_OK;
  }
  if (strcmp(name, "raster_n_group") == 0) {
    if (value < -1) return fail(FLCE_ERR_INVALID_ARGUMENT, "raster_n_group must be >= -1 (-1: chosen per GEMM, 0: all)");
    g_n_group = static_cast<int>(value);
    return FLCE_OK;
  }
  return fail(FLCE_ERR_INVALID_ARGUMENT, "unknown option '%s'", name);
}

size_t flce_b200_workspace_bytes(const flce_problem_t* p, int phase, size_t slab_budget_bytes) {
  if (check_problem(p) != FLCE_OK) return 0;
  {  // the planners size work for the device's SM count: make sure it is known (a host without a GPU plans for 148)
    DeviceState* dev = nullptr;
    (void)device_state(&dev);
  }
  if (phase == FLCE_PHASE_FORWARD) return forward_plan(p).total;
  if (phase == FLCE_PHASE_BACKWARD) return backward_plan(p, slab_budget_bytes, true).total;
  if (phase == FLCE_PHASE_FUSED) return fused_plan(p, slab_budget_bytes, true).total;
  if (phase == FLCE_PHASE_BACKWARD_SPLIT) {
    const BackwardPlan b = backward_plan(p, slab_budget_bytes, false);
    return b.coef_bytes + 2 * b.slab_bytes;
  }
  fail(FLCE_ERR_INVALID_ARGUMENT, "unknown phase %d", phase);
  return 0;
}

int flce_b200_count(const flce_problem_t* p, float* norm, void* stream) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (norm == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "norm is NULL");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  count_kernel<<<1, kRedThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(p->target), p->n_rows, p->ignore_index, p->ce_weight, p->vocab,
      p->vocab_offset, static_cast<float>(p->vocab_total), norm);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_forward_stats(const flce_problem_t* p, float* rowstats, void* workspace, size_t workspace_bytes,
                            void* stream_) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (rowstats == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "rowstats is NULL");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const ForwardPlan plan = forward_plan(p);
  if (workspace == nullptr || workspace_bytes < plan.total)
    return fail(FLCE_ERR_WORKSPACE, "forward needs %zu bytes of workspace, got %zu", plan.total, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const bool need_sum = p->label_smoothing > 0.f;
  StatsEpilogue::Params ep{};
  ep.target = reinterpret_cast<const long long*>(p->target);
  ep.bias = p->bias;
  ep.col_weight = p->ce_weight;
  ep.softcap = p->softcap;
  ep.inv_softcap = p->softcap > 0.f ? 1.f / p->softcap : 0.f;
  ep.n_cols = static_cast<int>(p->vocab);
  ep.vocab_offset = p->vocab_offset;
  ep.m_rows = static_cast<int>(p->n_rows);
  ep.pmax = reinterpret_cast<float*>(ws);
  ep.psum = reinterpret_cast<float*>(ws + plan.plane);
  ep.plogit_sum = need_sum ? reinterpret_cast<float*>(ws + 2 * plan.plane) : nullptr;
  const bool need_argmax = (p->flags & FLCE_FLAG_ARGMAX) != 0;
  ep.pamax_val = need_argmax ? reinterpret_cast<float*>(ws + 3 * plan.plane) : nullptr;
  ep.pamax_idx = need_argmax ? reinterpret_cast<int*>(ws + 4 * plan.plane) : nullptr;
  ep.target_logit = rowstats + 2 * static_cast<size_t>(p->n_rows);
  ep.logits_out = nullptr;
  ep.ld_logits = 0;
  ep.logits_fmt = kOutBf16;
  FLCE_CUDA(cudaMemsetAsync(ep.target_logit, 0, static_cast<size_t>(p->n_rows) * sizeof(float), stream));
  Operand a{p->x, p->n_rows, p->hidden, p->ld_x, 0};
  Operand b{p->w, p->vocab, p->hidden, p->ld_w, 0};
  rc = launch_gemm<kMajorK, kMajorK, StatsEpilogue>(*dev, kKindStats, g_cta_pair != 0, a, b, p->dtype, p->n_rows, p->vocab, p->hidden,
                                                    static_cast<long long>(kBlockM) * p->hidden * 2, false, ep, stream,
                                                    p->active_rows, 1);
  if (rc != FLCE_OK) return rc;
  const int threads = 256;
  merge_partials_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, threads)), threads, 0, stream>>>(
      static_cast<int>(p->n_rows), plan.n_tiles, ep.pmax, ep.psum, ep.plogit_sum, ep.pamax_val, ep.pamax_idx, rowstats);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

// ------------------------------------------------------------------ forward statistics without any allocation
// Scratch for flce_b200_forward_stats_static: lives in the library image, one copy per GPU that loads the library,
// for the life of the process.  In host code the array's name is only a handle; the device address comes from
// cudaGetSymbolAddress (once per device, below).
constexpr size_t kStaticScratchFloats = size_t(8) << 20;  // 8 Mi floats = 32 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static float* g_static_scratch_addr[64] = {nullptr};
static std::mutex g_static_scratch_mutex;

int flce_b200_forward_stats_static(const flce_problem_t* p, float* rowstats, void* stream_) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (rowstats == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "rowstats is NULL");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool need_sum = p->label_smoothing > 0.f;
  const bool need_argmax = (p->flags & FLCE_FLAG_ARGMAX) != 0;
  const size_t n_tiles = static_cast<size_t>(ceil_div(p->vocab, kBlockN));
  const size_t plane = align_up(n_tiles * static_cast<size_t>(p->n_rows), 64);  // floats; keeps planes 256-byte aligned
  const size_t n_planes = 2 + (need_sum ? 1 : 0) + (need_argmax ? 2 : 0);
  if (n_planes * plane > kStaticScratchFloats)
    return fail(FLCE_ERR_WORKSPACE,
                "problem too large for the built-in scratch: %zu planes x %zu vocabulary tiles x %lld rows = %zu floats, "
                "limit %zu floats (32 MiB); use flce_b200_forward_stats with caller-provided workspace",
                n_planes, n_tiles, (long long)p->n_rows, n_planes * plane, kStaticScratchFloats);
  // one-time set-up for the current device: resolve the array's device address
  int ordinal = 0;
  FLCE_CUDA(cudaGetDevice(&ordinal));
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[ordinal] == nullptr) {
      void* addr = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&addr, g_static_scratch);
      if (e != cudaSuccess || addr == nullptr)
        return fail(FLCE_ERR_CUDA, "cudaGetSymbolAddress(built-in scratch) failed on device %d: %s", ordinal,
                    cudaGetErrorString(e));
      g_static_scratch_addr[ordinal] = static_cast<float*>(addr);
    }
    scratch = g_static_scratch_addr[ordinal];
  }
  // Every (row, tile) entry that the merge below reads is written by the sweep first, so nothing in the shared
  // array has to start at zero; only the caller's target-logit plane does.
  size_t next = 0;
  StatsEpilogue::Params ep{};
  ep.target = reinterpret_cast<const long long*>(p->target);
  ep.bias = p->bias;
  ep.col_weight = p->ce_weight;
  ep.softcap = p->softcap;
  ep.inv_softcap = p->softcap > 0.f ? 1.f / p->softcap : 0.f;
  ep.n_cols = static_cast<int>(p->vocab);
  ep.vocab_offset = p->vocab_offset;
  ep.m_rows = static_cast<int>(p->n_rows);
  ep.pmax = scratch + plane * next++;
  ep.psum = scratch + plane * next++;
  ep.plogit_sum = need_sum ? scratch + plane * next++ : nullptr;
  ep.pamax_val = need_argmax ? scratch + plane * next++ : nullptr;
  ep.pamax_idx = need_argmax ? reinterpret_cast<int*>(scratch + plane * next++) : nullptr;
  ep.target_logit = rowstats + 2 * static_cast<size_t>(p->n_rows);
  ep.logits_out = nullptr;
  ep.ld_logits = 0;
  ep.logits_fmt = kOutBf16;
  FLCE_CUDA(cudaMemsetAsync(ep.target_logit, 0, static_cast<size_t>(p->n_rows) * sizeof(float), stream));
  Operand a{p->x, p->n_rows, p->hidden, p->ld_x, 0};
  Operand b{p->w, p->vocab, p->hidden, p->ld_w, 0};
  rc = launch_gemm<kMajorK, kMajorK, StatsEpilogue>(*dev, kKindStats, g_cta_pair != 0, a, b, p->dtype, p->n_rows, p->vocab,
                                                    p->hidden, static_cast<long long>(kBlockM) * p->hidden * 2, false, ep,
                                                    stream);
  if (rc != FLCE_OK) return rc;
  const int threads = 256;
  merge_partials_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, threads)), threads, 0, stream>>>(
      static_cast<int>(p->n_rows), static_cast<int>(n_tiles), ep.pmax, ep.psum, ep.plogit_sum, ep.pamax_val, ep.pamax_idx,
      rowstats);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_forward_finalize(const flce_problem_t* p, const float* rowstats, const float* norm,
                               const flce_forward_out_t* out, void* stream_) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (rowstats == nullptr || norm == nullptr || out == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "rowstats, norm and out must not be NULL");
  if (out->scalars != nullptr && out->loss_rows == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "scalars requires loss_rows");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int threads = 256;
  finalize_rows_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, threads)), threads, 0, stream>>>(
      static_cast<int>(p->n_rows), row_math(p), reinterpret_cast<const long long*>(p->target), p->ce_weight, rowstats,
      norm, out->lse, out->target_prob, out->loss_rows, out->z_loss_rows, out->correct_rows,
      reinterpret_cast<long long*>(out->predicted_tokens));
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  if (out->scalars != nullptr) {
    reduce_rows_kernel<<<1, kRedThreads, 0, stream>>>(static_cast<int>(p->n_rows), out->loss_rows, out->z_loss_rows,
                                                     out->correct_rows, norm, out->scalars);
    FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  }
  return FLCE_OK;
}

int flce_b200_forward(const flce_problem_t* p, float* norm, float* rowstats, const flce_forward_out_t* out,
                      void* workspace, size_t workspace_bytes, void* stream) {
  int rc = flce_b200_count(p, norm, stream);
  if (rc != FLCE_OK) return rc;
  rc = flce_b200_forward_stats(p, rowstats, workspace, workspace_bytes, stream);
  if (rc != FLCE_OK) return rc;
  return flce_b200_forward_finalize(p, rowstats, norm, out, stream);
}

int flce_b200_backward(const flce_problem_t* p, const flce_backward_args_t* args, void* workspace,
                       size_t workspace_bytes, size_t slab_budget_bytes, void* stream_) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (args == nullptr || args->lse == nullptr || args->norm == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "args, args->lse and args->norm must not be NULL");
  if (p->use_token_scaling && args->target_prob == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "token scaling needs target_prob from the forward pass");
  if (args->grad_dtype != p->dtype && args->grad_dtype != FLCE_FP32)
    return fail(FLCE_ERR_UNSUPPORTED, "gradients must be in the input dtype or fp32");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool grads_fp32 = args->grad_dtype == FLCE_FP32;
  // projection operands: by default the problem's own x and w; a caller that fed split high/low 16-bit terms of
  // fp32 tensors to the logits GEMM projects onto narrower term matrices instead
  const void* px = args->proj_x != nullptr ? args->proj_x : p->x;
  const long long px_cols = args->proj_x != nullptr ? args->proj_x_cols : p->hidden;
  const long long ld_px = args->proj_x != nullptr ? args->ld_proj_x : p->ld_x;
  const void* pw = args->proj_w != nullptr ? args->proj_w : p->w;
  const long long pw_cols = args->proj_w != nullptr ? args->proj_w_cols : p->hidden;
  const long long ld_pw = args->proj_w != nullptr ? args->ld_proj_w : p->ld_w;
  const bool split = args->split_logit_grad != 0;
  if (px_cols <= 0 || pw_cols <= 0 || px_cols % 8 != 0 || pw_cols % 8 != 0 || ld_px % 8 != 0 || ld_pw % 8 != 0 ||
      ld_px < px_cols || ld_pw < pw_cols)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "projection operands need column counts and pitches that are multiples of 8");
  if ((args->proj_x != nullptr || args->proj_w != nullptr || split) && !grads_fp32)
    return fail(FLCE_ERR_UNSUPPORTED, "projection operands and the split logit gradient need fp32 gradient outputs");
  if (split && (args->lo_cols_x <= 0 || args->lo_cols_x > px_cols || args->lo_cols_w <= 0 || args->lo_cols_w > pw_cols ||
                args->lo_cols_x % 8 != 0 || args->lo_cols_w % 8 != 0))
    return fail(FLCE_ERR_INVALID_ARGUMENT, "lo_cols_x / lo_cols_w must be positive multiples of 8 within the projection widths");
  const BackwardPlan plan = backward_plan(p, slab_budget_bytes, true);
  const size_t needed = plan.coef_bytes + plan.slab_bytes * (split ? 2 : 1) +
                        ((args->grad_input != nullptr && !grads_fp32) ? plan.acc_bytes : 0);
  if (workspace == nullptr || workspace_bytes < needed)
    return fail(FLCE_ERR_WORKSPACE, "backward needs %zu bytes of workspace, got %zu", needed, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* c1 = reinterpret_cast<float*>(ws);
  float* c2 = c1 + p->n_rows;
  float* c3 = c2 + p->n_rows;
  uint16_t* dz = reinterpret_cast<uint16_t*>(ws + plan.coef_bytes);
  uint16_t* dz_lo = split ? reinterpret_cast<uint16_t*>(ws + plan.coef_bytes + plan.slab_bytes) : nullptr;
  float* dx_acc = reinterpret_cast<float*>(ws + plan.coef_bytes + plan.slab_bytes);   // unused with fp32 gradients

  int slab_begin = args->slab_begin, slab_end = args->slab_end;
  if (slab_begin == 0 && slab_end == 0) slab_end = plan.n_slabs;
  if (slab_begin < 0 || slab_end > plan.n_slabs || slab_begin >= slab_end)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "slab range [%d, %d) outside the plan's %d slabs", slab_begin, slab_end,
                plan.n_slabs);
  const int threads = 256;
  coef_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, threads)), threads, 0, stream>>>(
      static_cast<int>(p->n_rows), row_math(p), reinterpret_cast<const long long*>(p->target), p->ce_weight, args->lse,
      args->target_prob, args->norm, args->grad_output, args->grad_output_per_row, c1, c2, c3);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;

  const bool pair = g_cta_pair != 0;
  const int esize_out = grads_fp32 ? 4 : 2;
  for (int s = slab_begin; s < slab_end; ++s) {
    const long long v0 = static_cast<long long>(s) * plan.slab_cols;
    const long long cols = (p->vocab - v0 < plan.slab_cols) ? p->vocab - v0 : plan.slab_cols;
    const uint16_t* w_slab = static_cast<const uint16_t*>(p->w) + v0 * p->ld_w;
    // ---- recompute logits of this slab -> dZ
    {
      DzEpilogue::Params ep;
      ep.target = reinterpret_cast<const long long*>(p->target);
      ep.bias = p->bias != nullptr ? p->bias + v0 : nullptr;
      ep.col_weight = p->ce_weight != nullptr ? p->ce_weight + v0 : nullptr;
      ep.softcap = p->softcap;
      ep.inv_softcap = p->softcap > 0.f ? 1.f / p->softcap : 0.f;
      ep.n_cols = static_cast<int>(cols);
      ep.vocab_offset = p->vocab_offset + v0;
      ep.m_rows = static_cast<int>(p->n_rows);
      ep.lse = args->lse;
      ep.c1 = c1;
      ep.c2 = c2;
      ep.c3 = c3;
      ep.dz = dz;
      ep.dz_lo = dz_lo;
      ep.ld_dz = plan.ld_dz;
      ep.out_fmt = p->dtype == FLCE_BF16 ? kOutBf16 : kOutFp16;
      Operand a{p->x, p->n_rows, p->hidden, p->ld_x, 0};
      Operand b{w_slab, cols, p->hidden, p->ld_w, 0};
      rc = launch_gemm<kMajorK, kMajorK, DzEpilogue>(*dev, kKindDz, pair, a, b, p->dtype, p->n_rows, cols, p->hidden,
                                                     static_cast<long long>(kBlockM) * p->hidden * 2, false, ep, stream,
                                                     p->active_rows, 1);
      if (rc != FLCE_OK) return rc;
    }
    // ---- grad_weight[slab] = dZ^T . X        (M = cols, N = hidden, K = n_rows; both operands MN-major)
    if (args->grad_weight != nullptr) {
      StoreEpilogue::Params ep{};
      ep.m_rows = static_cast<int>(cols);
      ep.n_cols = static_cast<int>(px_cols);
      ep.acc_in = nullptr;
      ep.acc_out = nullptr;
      ep.ld_acc = 0;
      ep.out = static_cast<uint8_t*>(args->grad_weight) + static_cast<size_t>(v0) * px_cols * esize_out;
      ep.ld_out = px_cols;
      ep.out_fmt = grads_fp32 ? kOutFp32 : (p->dtype == FLCE_BF16 ? kOutBf16 : kOutFp16);
      Operand a{dz, cols, p->n_rows, plan.ld_dz, 1};
      Operand b{px, px_cols, p->n_rows, ld_px, 1};
      rc = launch_gemm<kMajorMN, kMajorMN, StoreEpilogue>(*dev, kKindDw, pair, a, b, p->dtype, cols, px_cols, p->n_rows, 0, true,
                                                          ep, stream, p->active_rows, 2);
      if (rc != FLCE_OK) return rc;
      if (split) {  // rounding residual of dZ against the leading (high-order) columns of the projection operand
        float* acc = reinterpret_cast<float*>(ep.out);
        ep.n_cols = static_cast<int>(args->lo_cols_x);
        ep.acc_in = acc;
        ep.acc_out = acc;
        ep.ld_acc = px_cols;
        ep.out = nullptr;
        Operand a2{dz_lo, cols, p->n_rows, plan.ld_dz, 1};
        Operand b2{px, args->lo_cols_x, p->n_rows, ld_px, 1};
        rc = launch_gemm<kMajorMN, kMajorMN, StoreEpilogue>(*dev, kKindDw, pair, a2, b2, p->dtype, cols, args->lo_cols_x,
                                                            p->n_rows, 0, true, ep, stream, p->active_rows, 2);
        if (rc != FLCE_OK) return rc;
      }
    }
    // ---- grad_input (+)= dZ . W[slab]        (M = n_rows, N = hidden, K = cols; B is MN-major)
    if (args->grad_input != nullptr) {
      StoreEpilogue::Params ep{};
      ep.m_rows = static_cast<int>(p->n_rows);
      ep.n_cols = static_cast<int>(pw_cols);
      const bool first = s == 0, last = s == plan.n_slabs - 1;
      float* acc = grads_fp32 ? static_cast<float*>(args->grad_input) : dx_acc;
      ep.acc_in = first ? nullptr : acc;
      ep.acc_out = (last && !grads_fp32) ? nullptr : acc;
      if (plan.n_slabs == 1 && !grads_fp32) ep.acc_out = nullptr;
      ep.ld_acc = pw_cols;
      ep.out = (last && !grads_fp32) ? args->grad_input : nullptr;
      ep.ld_out = pw_cols;
      ep.out_fmt = p->dtype == FLCE_BF16 ? kOutBf16 : kOutFp16;
      const uint16_t* pw_slab = static_cast<const uint16_t*>(pw) + v0 * ld_pw;
      Operand a{dz, p->n_rows, cols, plan.ld_dz, 0};
      Operand b{pw_slab, pw_cols, cols, ld_pw, 1};
      rc = launch_gemm<kMajorK, kMajorMN, StoreEpilogue>(*dev, kKindDx, pair, a, b, p->dtype, p->n_rows, pw_cols, cols, 0, true,
                                                         ep, stream, p->active_rows, 1);
      if (rc != FLCE_OK) return rc;
      if (split) {
        ep.n_cols = static_cast<int>(args->lo_cols_w);
        ep.acc_in = acc;
        ep.acc_out = acc;
        ep.out = nullptr;
        Operand a2{dz_lo, p->n_rows, cols, plan.ld_dz, 0};
        Operand b2{pw_slab, args->lo_cols_w, cols, ld_pw, 1};
        rc = launch_gemm<kMajorK, kMajorMN, StoreEpilogue>(*dev, kKindDx, pair, a2, b2, p->dtype, p->n_rows, args->lo_cols_w,
                                                           cols, 0, true, ep, stream, p->active_rows, 1);
        if (rc != FLCE_OK) return rc;
      }
    }
    if (args->grad_bias != nullptr) {
      colsum_kernel<<<static_cast<unsigned>(ceil_div(cols, 64)), 1024, 0, stream>>>(
          dz, plan.ld_dz, static_cast<int>(p->n_rows), static_cast<int>(cols), p->dtype == FLCE_BF16 ? kOutBf16 : kOutFp16,
          args->grad_bias + v0, p->active_rows);
      FLCE_CUDA(cudaGetLastError());
      ++g_kernel_launches;
      if (split) {
        colsum_accumulate_kernel<<<static_cast<unsigned>(ceil_div(cols, 64)), 1024, 0, stream>>>(
            dz_lo, plan.ld_dz, static_cast<int>(p->n_rows), static_cast<int>(cols),
            p->dtype == FLCE_BF16 ? kOutBf16 : kOutFp16, args->grad_bias + v0, 1, p->active_rows);
        FLCE_CUDA(cudaGetLastError());
        ++g_kernel_launches;
      }
    }
  }
  return FLCE_OK;
}

// out[c] (+)= sum_r scale[r] * mat[r, c] in two ordered stages (row_kernels.cuh)
static int launch_scaled_colsum(const void* mat, long long ld, long long n_rows, long long n_cols, int fmt, const float* scale,
                                float* scratch, float* out, bool accumulate, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(ceil_div(n_cols, 64)), kColsumSplits, 1);
  scaled_colsum_stage1_kernel<<<grid, 1024, 0, stream>>>(static_cast<const uint16_t*>(mat), ld, static_cast<int>(n_rows),
                                                         static_cast<int>(n_cols), fmt, scale, scratch);
  FLCE_CUDA(cudaGetLastError());
  scaled_colsum_stage2_kernel<<<static_cast<unsigned>(ceil_div(n_cols, 256)), 256, 0, stream>>>(
      scratch, static_cast<int>(n_cols), out, accumulate ? 1 : 0);
  FLCE_CUDA(cudaGetLastError());
  g_kernel_launches += 2;
  return FLCE_OK;
}

int flce_b200_forward_backward(const flce_problem_t* p, const flce_fused_args_t* args, void* workspace,
                               size_t workspace_bytes, size_t slab_budget_bytes, void* stream_) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (args == nullptr || args->out == nullptr || args->norm == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "args, args->out and args->norm must not be NULL");
  const flce_forward_out_t* out = args->out;
  if (out->lse == nullptr || out->loss_rows == nullptr || out->target_prob == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "single-sweep mode needs out->lse, out->target_prob and out->loss_rows");
  if (p->reduction == FLCE_NONE)
    return fail(FLCE_ERR_UNSUPPORTED, "single-sweep mode forms gradients before the upstream gradient is known; "
                                      "reduction 'none' needs the two-sweep path");
  const bool sharded = p->vocab != p->vocab_total || p->vocab_offset != 0;
  if (sharded && (args->exchange_shift == nullptr || args->exchange_rowstats == nullptr || args->after_grad_input == nullptr))
    return fail(FLCE_ERR_UNSUPPORTED, "a vocabulary shard does not know a row's log-sum-exp on its own: single-sweep mode "
                                      "needs the three exchange hooks of flce_fused_args_t there (or use the two-sweep path)");
  if (sharded && args->grad_bias != nullptr)
    return fail(FLCE_ERR_UNSUPPORTED, "grad_bias is not formed on a vocabulary shard");
  if (args->grad_dtype != p->dtype && args->grad_dtype != FLCE_FP32)
    return fail(FLCE_ERR_UNSUPPORTED, "gradients must be in the input dtype or fp32");
  if (args->store_mode < FLCE_STORE_AUTO || args->store_mode > FLCE_STORE_EXP)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "bad store_mode %d", args->store_mode);
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool grads_fp32 = args->grad_dtype == FLCE_FP32;
  const bool smoothing = p->label_smoothing > 0.f;
  // The exp-store form covers everything whose logit gradient is (per-row factor) x (stored value) plus rank-1 terms:
  // not the uniform smoothing term under a soft-cap (its chain factor varies per element), and not the bias gradient
  // (a column sum of the scaled gradient, which this form never materialises).  It needs bf16's exponent range:
  // exp(s - shift) spans e^-87 .. e^60 here, fp16 holds e^-16 .. e^11.
  const bool exp_ok = !(smoothing && p->softcap > 0.f) && args->grad_bias == nullptr && p->dtype == FLCE_BF16;
  if (args->store_mode == FLCE_STORE_EXP && !exp_ok)
    return fail(FLCE_ERR_UNSUPPORTED, "the exp-store form needs bf16 operands and does not cover label smoothing together "
                                      "with a soft-cap, nor grad_bias");
  const bool exp_store = args->store_mode == FLCE_STORE_LOGITS ? false : exp_ok;
  const FusedPlan plan = fused_plan(p, slab_budget_bytes, true);
  const bool use_acc = args->grad_weight != nullptr && !grads_fp32 && plan.n_chunks > 1;
  const size_t needed = plan.total - (use_acc ? 0 : plan.acc_bytes);
  if (workspace == nullptr || workspace_bytes < needed)
    return fail(FLCE_ERR_WORKSPACE, "single-sweep mode needs %zu bytes of workspace, got %zu", needed, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  size_t at = 0;
  auto carve = [&](size_t bytes) { uint8_t* ptr = ws + at; at += bytes; return ptr; };
  float* planes = reinterpret_cast<float*>(carve(5 * plan.plane));
  float* chunk_stats = reinterpret_cast<float*>(carve(plan.rowstats_bytes));
  float* c1 = reinterpret_cast<float*>(carve(plan.coef_bytes));
  uint16_t* slab = reinterpret_cast<uint16_t*>(carve(plan.slab_bytes));
  float* shift = reinterpret_cast<float*>(carve(plan.shift_bytes));
  float* alpha = reinterpret_cast<float*>(carve(plan.alpha_bytes));
  uint16_t* xs = reinterpret_cast<uint16_t*>(carve(plan.xs_bytes));
  float* w_sum = reinterpret_cast<float*>(carve(plan.vec_bytes));     // sum_j w_j W[j, :]
  float* x_sum = reinterpret_cast<float*>(carve(plan.vec_bytes));     // sum_r c2_r x[r, :]
  float* colsum_scratch = reinterpret_cast<float*>(carve(plan.colsum_scratch_bytes));
  int* redo_flags = reinterpret_cast<int*>(carve(plan.flag_bytes));     // one per chunk: sweep 1 again with shift = lse
  float* dw_acc = reinterpret_cast<float*>(carve(0));                  // last: present only when use_acc

  if (!args->norm_given) {
    rc = flce_b200_count(p, args->norm, stream_);
    if (rc != FLCE_OK) return rc;
  }
  const bool pair = g_cta_pair != 0;
  const bool need_sum = smoothing;
  const bool need_argmax = (p->flags & FLCE_FLAG_ARGMAX) != 0;
  const int fmt16 = p->dtype == FLCE_BF16 ? kOutBf16 : kOutFp16;
  const int esize_out = grads_fp32 ? 4 : 2;
  const RowMath rm = row_math(p);
  const int threads = 256;
  const size_t plane_floats = plan.plane / sizeof(float);
  const float inv_softcap = p->softcap > 0.f ? 1.f / p->softcap : 0.f;
  const long long* target_all = reinterpret_cast<const long long*>(p->target);
  if (exp_store) {
    FLCE_CUDA(cudaMemsetAsync(redo_flags, 0, plan.flag_bytes, stream));
    const int warps = 8;
    target_shift_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, warps)), warps * 32, 0, stream>>>(
        static_cast<const uint16_t*>(p->x), p->ld_x, static_cast<const uint16_t*>(p->w), p->ld_w, fmt16,
        static_cast<int>(p->n_rows), static_cast<int>(p->hidden), target_all, p->ignore_index, p->vocab, p->vocab_offset,
        sharded ? 1 : 0, p->bias, p->softcap, inv_softcap, kExpStoreOffset, shift);
    FLCE_CUDA(cudaGetLastError());
    ++g_kernel_launches;
    if (sharded) {
      args->exchange_shift(args->exchange_user, shift, p->n_rows);
      shift_fill_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, threads)), threads, 0, stream>>>(
          static_cast<int>(p->n_rows), kExpStoreOffset, shift);
      FLCE_CUDA(cudaGetLastError());
      ++g_kernel_launches;
    }
    if (smoothing && args->grad_input != nullptr) {
      rc = launch_scaled_colsum(p->w, p->ld_w, p->vocab, p->hidden, fmt16, p->ce_weight, colsum_scratch, w_sum, false, stream);
      if (rc != FLCE_OK) return rc;
    }
  }
  for (int c = 0; c < plan.n_chunks; ++c) {
    const long long r0 = static_cast<long long>(c) * plan.chunk_rows;
    const long long rows = (p->n_rows - r0 < plan.chunk_rows) ? p->n_rows - r0 : plan.chunk_rows;
    const uint16_t* x_chunk = static_cast<const uint16_t*>(p->x) + r0 * p->ld_x;
    const long long* tgt = target_all + r0;
    const int base = static_cast<int>(r0);
    float* c2 = c1 + rows;
    float* c3 = c2 + rows;
    const bool first = c == 0, last = c == plan.n_chunks - 1;
    // ---- logits of the chunk: statistics + 16-bit copy (the logits themselves, or their exponentials)
    auto sweep1 = [&](const int* gate) -> int {
      StatsEpilogue::Params ep{};
      ep.target = tgt;
      ep.bias = p->bias;
      ep.col_weight = p->ce_weight;
      ep.softcap = p->softcap;
      ep.inv_softcap = inv_softcap;
      ep.n_cols = static_cast<int>(p->vocab);
      ep.vocab_offset = p->vocab_offset;
      ep.m_rows = static_cast<int>(rows);
      ep.pmax = planes;
      ep.psum = planes + plane_floats;
      ep.plogit_sum = need_sum ? planes + 2 * plane_floats : nullptr;
      ep.pamax_val = need_argmax ? planes + 3 * plane_floats : nullptr;
      ep.pamax_idx = need_argmax ? reinterpret_cast<int*>(planes + 4 * plane_floats) : nullptr;
      ep.target_logit = chunk_stats + 2 * static_cast<size_t>(rows);
      ep.logits_out = slab;
      ep.ld_logits = plan.ld_slab;
      ep.logits_fmt = fmt16;
      ep.shift = exp_store ? shift + r0 : nullptr;
      ep.ignore_index = p->ignore_index;
      if (gate == nullptr)   // (the gated repeat writes the same target logits again)
        FLCE_CUDA(cudaMemsetAsync(ep.target_logit, 0, static_cast<size_t>(rows) * sizeof(float), stream));
      Operand a{x_chunk, rows, p->hidden, p->ld_x, 0};
      Operand b{p->w, p->vocab, p->hidden, p->ld_w, 0};
      int rc1 = launch_gemm<kMajorK, kMajorK, StatsEpilogue>(*dev, kKindStats, pair, a, b, p->dtype, rows, p->vocab, p->hidden,
                                                             static_cast<long long>(kBlockM) * p->hidden * 2, false, ep, stream,
                                                             p->active_rows, 1, base, gate);
      if (rc1 != FLCE_OK) return rc1;
      if (gate == nullptr) {
        merge_partials_kernel<<<static_cast<unsigned>(ceil_div(rows, threads)), threads, 0, stream>>>(
            static_cast<int>(rows), plan.n_tiles, ep.pmax, ep.psum, ep.plogit_sum, ep.pamax_val, ep.pamax_idx, chunk_stats);
        FLCE_CUDA(cudaGetLastError());
        ++g_kernel_launches;
      }
      return FLCE_OK;
    };
    rc = sweep1(nullptr);
    if (rc != FLCE_OK) return rc;
    if (sharded) args->exchange_rowstats(args->exchange_user, chunk_stats, rows, r0);
    // ---- per-row losses, then the gradient coefficients (upstream gradient = 1)
    finalize_rows_kernel<<<static_cast<unsigned>(ceil_div(rows, threads)), threads, 0, stream>>>(
        static_cast<int>(rows), rm, tgt, p->ce_weight, chunk_stats, args->norm, out->lse + r0, out->target_prob + r0,
        out->loss_rows + r0, out->z_loss_rows != nullptr ? out->z_loss_rows + r0 : nullptr,
        out->correct_rows != nullptr ? out->correct_rows + r0 : nullptr,
        out->predicted_tokens != nullptr ? reinterpret_cast<long long*>(out->predicted_tokens) + r0 : nullptr);
    FLCE_CUDA(cudaGetLastError());
    ++g_kernel_launches;
    coef_kernel<<<static_cast<unsigned>(ceil_div(rows, threads)), threads, 0, stream>>>(
        static_cast<int>(rows), rm, tgt, p->ce_weight, out->lse + r0, out->target_prob + r0, args->norm, nullptr, 0, c1, c2, c3);
    FLCE_CUDA(cudaGetLastError());
    ++g_kernel_launches;
    if (exp_store) {
      // ---- a row further from its reference point than the stored form can express sends the chunk through sweep 1 again
      exp_store_check_kernel<<<static_cast<unsigned>(ceil_div(rows, threads)), threads, 0, stream>>>(
          static_cast<int>(rows), tgt, p->ignore_index, out->lse + r0, shift + r0, kExpStoreRedoLimit,
          redo_flags + c);
      FLCE_CUDA(cudaGetLastError());
      exp_store_reshift_kernel<<<static_cast<unsigned>(ceil_div(rows, threads)), threads, 0, stream>>>(
          static_cast<int>(rows), out->lse + r0, redo_flags + c, shift + r0);
      FLCE_CUDA(cudaGetLastError());
      g_kernel_launches += 2;
      rc = sweep1(redo_flags + c);
      if (rc != FLCE_OK) return rc;
      // ---- per-row factor, scaled copy of x, true-class entries of E
      ProfileSlot* slot = profile_begin(kKindOther, stream);
      exp_store_fixup_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(
          x_chunk, p->ld_x, static_cast<int>(p->hidden), fmt16, static_cast<int>(rows), tgt, p->ignore_index, p->vocab,
          p->vocab_offset, out->lse + r0, shift + r0, chunk_stats + 2 * static_cast<size_t>(rows), c1, c3, inv_softcap, kExpStoreClamp, slab,
          plan.ld_slab, alpha, xs, p->hidden);
      profile_end(slot, stream);
      FLCE_CUDA(cudaGetLastError());
      ++g_kernel_launches;
      if (smoothing && args->grad_weight != nullptr) {
        rc = launch_scaled_colsum(x_chunk, p->ld_x, rows, p->hidden, fmt16, c2, colsum_scratch, x_sum, !first, stream);
        if (rc != FLCE_OK) return rc;
      }
    } else {
      // ---- logits -> logit gradient, in place
      dim3 grid(static_cast<unsigned>(ceil_div(p->vocab, kDzInplaceCols)), static_cast<unsigned>(rows), 1);
      ProfileSlot* slot = profile_begin(kKindOther, stream);
      dz_inplace_kernel<<<grid, kDzInplaceThreads, 0, stream>>>(slab, plan.ld_slab, static_cast<int>(rows),
                                                                static_cast<int>(p->vocab), fmt16, tgt, p->vocab_offset,
                                                                out->lse + r0, c1, c2, c3, p->ce_weight, inv_softcap,
                                                                p->active_rows, base);
      profile_end(slot, stream);
      FLCE_CUDA(cudaGetLastError());
      ++g_kernel_launches;
    }
    // ---- grad_input[chunk] = dZ . W          (M = rows, N = hidden, K = vocab; B is MN-major)
    auto grad_input_gemm = [&](int reserve_sms) -> int {
      if (args->grad_input == nullptr) return FLCE_OK;
      StoreEpilogue::Params ep{};
      ep.m_rows = static_cast<int>(rows);
      ep.n_cols = static_cast<int>(p->hidden);
      ep.out = static_cast<uint8_t*>(args->grad_input) + static_cast<size_t>(r0) * p->hidden * esize_out;
      ep.ld_out = p->hidden;
      ep.out_fmt = grads_fp32 ? kOutFp32 : fmt16;
      if (exp_store) {
        ep.row_scale = alpha;
        if (smoothing) {
          ep.r1_row = c2;
          ep.r1_col = w_sum;
        }
      }
      Operand a{slab, rows, p->vocab, plan.ld_slab, 0};
      Operand b{p->w, p->hidden, p->vocab, p->ld_w, 1};
      return launch_gemm<kMajorK, kMajorMN, StoreEpilogue>(*dev, kKindDx, pair, a, b, p->dtype, rows, p->hidden, p->vocab, 0, true,
                                                           ep, stream, p->active_rows, 1, base, nullptr, reserve_sms);
    };
    // ---- grad_weight (+)= dZ^T . X[chunk]    (M = vocab, N = hidden, K = rows; both operands MN-major)
    auto grad_weight_gemm = [&](int reserve_sms) -> int {
      if (args->grad_weight == nullptr) return FLCE_OK;
      StoreEpilogue::Params ep{};
      ep.m_rows = static_cast<int>(p->vocab);
      ep.n_cols = static_cast<int>(p->hidden);
      // One chunk: written once in the final dtype.  Several: the first chunk stores its fp32 part, the others add theirs
      // with reductions at L2 (no read-modify-write in the epilogue), and a 16-bit result is converted after the last.
      float* acc = grads_fp32 ? static_cast<float*>(args->grad_weight) : dw_acc;
      const bool direct = plan.n_chunks == 1 && !grads_fp32;
      ep.acc_in = nullptr;
      ep.acc_out = direct ? nullptr : acc;
      ep.acc_add = (!direct && !first) ? 1 : 0;
      ep.ld_acc = p->hidden;
      ep.out = direct ? args->grad_weight : nullptr;
      ep.ld_out = p->hidden;
      ep.out_fmt = fmt16;
      if (exp_store && smoothing && last) {   // the uniform term of every chunk at once: - w_j * sum_r c2_r x_r
        ep.r1_row = p->ce_weight;
        ep.r1_col = x_sum;
      }
      Operand a{slab, p->vocab, rows, plan.ld_slab, 1};
      Operand b{exp_store ? static_cast<const void*>(xs) : static_cast<const void*>(x_chunk), p->hidden, rows,
                exp_store ? p->hidden : p->ld_x, 1};
      int rc2 = launch_gemm<kMajorMN, kMajorMN, StoreEpilogue>(*dev, kKindDw, pair, a, b, p->dtype, p->vocab, p->hidden, rows, 0,
                                                               true, ep, stream, p->active_rows, 2, base, nullptr, reserve_sms);
      if (rc2 != FLCE_OK) return rc2;
      if (last && !direct && !grads_fp32) {
        ProfileSlot* slot = profile_begin(kKindOther, stream);
        convert_f32_kernel<<<dev->sm_count * 8, 256, 0, stream>>>(acc, static_cast<long long>(p->vocab) * p->hidden, fmt16,
                                                                   static_cast<uint16_t*>(args->grad_weight));
        profile_end(slot, stream);
        FLCE_CUDA(cudaGetLastError());
        ++g_kernel_launches;
      }
      return FLCE_OK;
    };
    if (last && args->after_grad_weight != nullptr) {
      // grad_weight is complete after this launch: let the caller enqueue what consumes it (an all-reduce on another
      // stream), then form the last chunk's grad_input beside it on the SMs that are left
      rc = grad_weight_gemm(0);
      if (rc != FLCE_OK) return rc;
      args->after_grad_weight(args->after_grad_weight_user);
      rc = grad_input_gemm(args->reserve_sms > 0 ? args->reserve_sms : 0);
      if (rc != FLCE_OK) return rc;
    } else {
      rc = grad_input_gemm(0);
      if (rc != FLCE_OK) return rc;
      int reserve = 0;
      if (sharded && args->grad_input != nullptr) {   // this shard's partial rows are on their way: let the caller start their sum
        args->after_grad_input(args->exchange_user,
                               static_cast<uint8_t*>(args->grad_input) + static_cast<size_t>(r0) * p->hidden * esize_out, rows, r0);
        reserve = args->reserve_sms > 0 ? args->reserve_sms : 0;
      }
      rc = grad_weight_gemm(reserve);
      if (rc != FLCE_OK) return rc;
    }
    if (args->grad_bias != nullptr) {
      colsum_accumulate_kernel<<<static_cast<unsigned>(ceil_div(p->vocab, 64)), 1024, 0, stream>>>(
          slab, plan.ld_slab, static_cast<int>(rows), static_cast<int>(p->vocab), fmt16, args->grad_bias, c != 0,
          p->active_rows, base);
      FLCE_CUDA(cudaGetLastError());
      ++g_kernel_launches;
    }
  }
  if (out->scalars != nullptr) {
    reduce_rows_kernel<<<1, kRedThreads, 0, stream>>>(static_cast<int>(p->n_rows), out->loss_rows, out->z_loss_rows,
                                                     out->correct_rows, args->norm, out->scalars);
    FLCE_CUDA(cudaGetLastError());
    ++g_kernel_launches;
  }
  return FLCE_OK;
}

int flce_b200_ce_forward(const flce_ce_problem_t* p, float* norm, float* rowstats, const flce_forward_out_t* out,
                         void* stream_) {
  int rc = check_ce_problem(p);
  if (rc != FLCE_OK) return rc;
  if (norm == nullptr || rowstats == nullptr || out == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "norm, rowstats and out must not be NULL");
  if (out->scalars != nullptr && out->loss_rows == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "scalars requires loss_rows");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long* tgt = reinterpret_cast<const long long*>(p->target);
  count_kernel<<<1, kRedThreads, 0, stream>>>(tgt, p->n_rows, p->ignore_index, p->ce_weight, p->vocab, 0,
                                             static_cast<float>(p->vocab), norm);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  if (p->dtype == FLCE_FP32) launch_ce_stats<float>(p, rowstats, stream);
  else if (p->dtype == FLCE_BF16) launch_ce_stats<__nv_bfloat16>(p, rowstats, stream);
  else launch_ce_stats<__half>(p, rowstats, stream);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  const int threads = 256;
  finalize_rows_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, threads)), threads, 0, stream>>>(
      static_cast<int>(p->n_rows), ce_row_math(p), tgt, p->ce_weight, rowstats, norm, out->lse, out->target_prob,
      out->loss_rows, out->z_loss_rows, out->correct_rows, reinterpret_cast<long long*>(out->predicted_tokens));
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  if (out->scalars != nullptr) {
    reduce_rows_kernel<<<1, kRedThreads, 0, stream>>>(static_cast<int>(p->n_rows), out->loss_rows, out->z_loss_rows,
                                                     out->correct_rows, norm, out->scalars);
    FLCE_CUDA(cudaGetLastError());
    ++g_kernel_launches;
  }
  return FLCE_OK;
}

int flce_b200_ce_backward(const flce_ce_problem_t* p, const float* lse, const float* norm, const float* grad_output,
                          int32_t grad_output_per_row, void* grad_logits, int64_t ld_grad, float* coef_scratch,
                          void* stream_) {
  int rc = check_ce_problem(p);
  if (rc != FLCE_OK) return rc;
  if (lse == nullptr || norm == nullptr || grad_logits == nullptr || coef_scratch == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "lse, norm, grad_logits and coef_scratch must not be NULL");
  if (ld_grad < p->vocab) return fail(FLCE_ERR_INVALID_ARGUMENT, "ld_grad smaller than vocab");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  float* c1 = coef_scratch;
  float* c2 = c1 + p->n_rows;
  float* c3 = c2 + p->n_rows;
  const int threads = 256;
  coef_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, threads)), threads, 0, stream>>>(
      static_cast<int>(p->n_rows), ce_row_math(p), reinterpret_cast<const long long*>(p->target), p->ce_weight, lse, nullptr,
      norm, grad_output, grad_output_per_row, c1, c2, c3);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  if (p->dtype == FLCE_FP32) launch_ce_grad<float>(p, grad_logits, ld_grad, lse, c1, c2, c3, stream);
  else if (p->dtype == FLCE_BF16) launch_ce_grad<__nv_bfloat16>(p, grad_logits, ld_grad, lse, c1, c2, c3, stream);
  else launch_ce_grad<__half>(p, grad_logits, ld_grad, lse, c1, c2, c3, stream);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_ce_forward_backward(const flce_ce_problem_t* p, float* norm, float* rowstats, const flce_forward_out_t* out,
                                  void* grad_logits, int64_t ld_grad, void* stream_) {
  int rc = check_ce_problem(p);
  if (rc != FLCE_OK) return rc;
  if (norm == nullptr || rowstats == nullptr || out == nullptr || grad_logits == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "norm, rowstats, out and grad_logits must not be NULL");
  if (out->scalars != nullptr && out->loss_rows == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "scalars requires loss_rows");
  if (ld_grad < p->vocab) return fail(FLCE_ERR_INVALID_ARGUMENT, "ld_grad smaller than vocab");
  const long long esize = p->dtype == FLCE_FP32 ? 4 : 2;
  int cluster = 0, slice_vecs = 0;
  if (!ce_fused_geometry(p->vocab, esize, &cluster, &slice_vecs))
    return fail(FLCE_ERR_UNSUPPORTED,
                "row of %lld elements does not fit a cluster's shared memory or is not a multiple of 16 bytes: use the "
                "two-pass entry points", (long long)p->vocab);
  if (!ce_rows_vectorisable(p->logits, p->ld, p->dtype) || !ce_rows_vectorisable(grad_logits, ld_grad, p->dtype))
    return fail(FLCE_ERR_UNSUPPORTED, "logits / gradient rows are not 16-byte aligned: use the two-pass entry points");
  if (p->n_rows * cluster > 0x7fffffffll) return fail(FLCE_ERR_UNSUPPORTED, "too many rows for one launch");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long* tgt = reinterpret_cast<const long long*>(p->target);
  count_kernel<<<1, kRedThreads, 0, stream>>>(tgt, p->n_rows, p->ignore_index, p->ce_weight, p->vocab, 0,
                                             static_cast<float>(p->vocab), norm);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  CeFusedOut fo;
  fo.rowstats = rowstats;
  fo.lse = out->lse;
  fo.target_prob = out->target_prob;
  fo.loss_rows = out->loss_rows;
  fo.z_rows = out->z_loss_rows;
  fo.correct_rows = out->correct_rows;
  fo.predicted = reinterpret_cast<long long*>(out->predicted_tokens);
  // without a soft-cap the exponentials of the statistics pass are kept and reused for the gradient
  const bool store_exp = !(p->softcap > 0.f) && g_ce_store_exp.load() != 0;
  auto launch = [&](auto tag) {
    using T = decltype(tag);
    if (g_ce_warps.load() == 16)
      return store_exp ? launch_ce_fused<T, true, 16>(p, grad_logits, ld_grad, norm, fo, cluster, slice_vecs, *dev, stream)
                       : launch_ce_fused<T, false, 16>(p, grad_logits, ld_grad, norm, fo, cluster, slice_vecs, *dev, stream);
    return store_exp ? launch_ce_fused<T, true, 8>(p, grad_logits, ld_grad, norm, fo, cluster, slice_vecs, *dev, stream)
                     : launch_ce_fused<T, false, 8>(p, grad_logits, ld_grad, norm, fo, cluster, slice_vecs, *dev, stream);
  };
  if (p->dtype == FLCE_FP32) rc = launch(float{});
  else if (p->dtype == FLCE_BF16) rc = launch(__nv_bfloat16{});
  else rc = launch(__half{});
  if (rc != FLCE_OK) return rc;
  ++g_kernel_launches;
  if (out->scalars != nullptr) {
    reduce_rows_kernel<<<1, kRedThreads, 0, stream>>>(static_cast<int>(p->n_rows), out->loss_rows, out->z_loss_rows,
                                                     out->correct_rows, norm, out->scalars);
    FLCE_CUDA(cudaGetLastError());
    ++g_kernel_launches;
  }
  return FLCE_OK;
}

int flce_b200_ce_scale_gradient(void* grad_logits, int64_t ld_grad, int64_t n_rows, int64_t vocab, int32_t dtype,
                                const float* grad_output, int32_t grad_output_per_row, void* stream_) {
  if (grad_logits == nullptr || grad_output == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL argument");
  if (n_rows <= 0 || vocab <= 0 || ld_grad < vocab || n_rows > 0x7fffffffll || vocab > 0x7fffffffll)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "bad gradient shape (n_rows=%lld vocab=%lld ld=%lld)", (long long)n_rows,
                (long long)vocab, (long long)ld_grad);
  if (dtype < FLCE_BF16 || dtype > FLCE_FP32) return fail(FLCE_ERR_UNSUPPORTED, "gradient must be bf16, fp16 or fp32");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long per_thread = dtype == FLCE_FP32 ? 4 : 8;
  DeviceState* dev = nullptr;
  const int rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  const long long items = n_rows * ceil_div(ceil_div(vocab, per_thread), 256);
  const long long resident = static_cast<long long>(dev->sm_count) * 8;      // eight 256-thread blocks per SM
  dim3 grid(static_cast<unsigned>(items < resident ? items : resident), 1, 1);
  if (dtype == FLCE_FP32)
    ce_scale_gradient_kernel<float><<<grid, 256, 0, stream>>>(static_cast<float*>(grad_logits), ld_grad, static_cast<int>(n_rows),
                                                             static_cast<int>(vocab), grad_output, grad_output_per_row);
  else if (dtype == FLCE_BF16)
    ce_scale_gradient_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(grad_logits), ld_grad,
                                                                     static_cast<int>(n_rows), static_cast<int>(vocab),
                                                                     grad_output, grad_output_per_row);
  else
    ce_scale_gradient_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<__half*>(grad_logits), ld_grad, static_cast<int>(n_rows),
                                                              static_cast<int>(vocab), grad_output, grad_output_per_row);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_split_fp32(const float* src, int64_t rows, int64_t cols, int64_t ld_src, void* dst, int64_t ld_dst,
                         int64_t block_cols, const int32_t* pattern, int32_t n_blocks, int32_t dst_dtype, void* stream_) {
  if (src == nullptr || dst == nullptr || pattern == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL argument");
  if (rows <= 0 || cols <= 0 || block_cols < cols || n_blocks < 1 || n_blocks > 8 || ld_dst < block_cols * n_blocks)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "bad split shape (rows %lld cols %lld block_cols %lld blocks %d ld_dst %lld)",
                (long long)rows, (long long)cols, (long long)block_cols, n_blocks, (long long)ld_dst);
  if (dst_dtype != FLCE_BF16 && dst_dtype != FLCE_FP16) return fail(FLCE_ERR_UNSUPPORTED, "terms must be bf16 or fp16");
  if (rows > 65535) return fail(FLCE_ERR_INVALID_ARGUMENT, "split_fp32 handles at most 65535 rows per call");
  SplitPattern pat;
  for (int b = 0; b < 8; ++b) {
    pat.term[b] = b < n_blocks ? pattern[b] : 0;
    if (pat.term[b] < 0 || pat.term[b] > 2) return fail(FLCE_ERR_INVALID_ARGUMENT, "pattern entries must be 0, 1 or 2");
  }
  dim3 grid(static_cast<unsigned>(ceil_div(block_cols, 256)), static_cast<unsigned>(rows), 1);
  split_fp32_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_)>>>(src, rows, cols, ld_src, static_cast<uint16_t*>(dst),
                                                                       ld_dst, block_cols, pat, n_blocks,
                                                                       dst_dtype == FLCE_BF16 ? kOutBf16 : kOutFp16);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_compact_rows(const flce_problem_t* p, void* x_compact, int64_t* target_compact, int32_t* perm,
                           int32_t* active_rows, void* stream_) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (x_compact == nullptr || target_compact == nullptr || perm == nullptr || active_rows == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL output");
  if ((reinterpret_cast<uintptr_t>(x_compact) & 15) != 0 || (reinterpret_cast<uintptr_t>(p->x) & 15) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "x and x_compact must be 16-byte aligned");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  compact_plan_kernel<<<1, kRedThreads, 0, stream>>>(reinterpret_cast<const long long*>(p->target), static_cast<int>(p->n_rows),
                                                    p->ignore_index, perm, active_rows);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  gather_rows_kernel<<<static_cast<unsigned>(p->n_rows), 256, 0, stream>>>(
      static_cast<const uint8_t*>(p->x), p->ld_x * 2, perm, static_cast<uint8_t*>(x_compact), p->hidden * 2,
      reinterpret_cast<const long long*>(p->target), reinterpret_cast<long long*>(target_compact));
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_compact_rows_rmsnorm(const flce_problem_t* p, const void* gamma, float eps, float offset, int32_t casting_mode,
                                   void* x_compact, int64_t* target_compact, int32_t* perm, int32_t* active_rows, float* rstd,
                                   void* stream_) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  rc = check_rmsnorm(p->dtype, p->hidden, casting_mode, gamma);
  if (rc != FLCE_OK) return rc;
  if (x_compact == nullptr || target_compact == nullptr || perm == nullptr || active_rows == nullptr || rstd == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL output");
  if ((reinterpret_cast<uintptr_t>(x_compact) & 15) != 0 || (reinterpret_cast<uintptr_t>(p->x) & 15) != 0 || p->ld_x % 8 != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "x and x_compact must be 16-byte aligned with a row pitch that is a multiple of 8");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  compact_plan_kernel<<<1, kRedThreads, 0, stream>>>(reinterpret_cast<const long long*>(p->target), static_cast<int>(p->n_rows),
                                                    p->ignore_index, perm, active_rows);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  const unsigned grid = static_cast<unsigned>(p->n_rows);
  const long long* tgt = reinterpret_cast<const long long*>(p->target);
  long long* tgt_out = reinterpret_cast<long long*>(target_compact);
  if (p->dtype == FLCE_BF16)
    rmsnorm_gather_rows_kernel<__nv_bfloat16><<<grid, kRmsThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(p->x), p->ld_x, perm, static_cast<__nv_bfloat16*>(x_compact), p->hidden,
        static_cast<int>(p->hidden), static_cast<const __nv_bfloat16*>(gamma), eps, offset, casting_mode, rstd, tgt, tgt_out);
  else
    rmsnorm_gather_rows_kernel<__half><<<grid, kRmsThreads, 0, stream>>>(
        static_cast<const __half*>(p->x), p->ld_x, perm, static_cast<__half*>(x_compact), p->hidden, static_cast<int>(p->hidden),
        static_cast<const __half*>(gamma), eps, offset, casting_mode, rstd, tgt, tgt_out);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int64_t flce_b200_rmsnorm_partial_floats(int64_t hidden) {
  {  // make sure the device's SM count is known (a host without a GPU plans for 148)
    DeviceState* dev = nullptr;
    (void)device_state(&dev);
  }
  return hidden > 0 ? static_cast<int64_t>(rmsnorm_partial_blocks()) * hidden : 0;
}

int flce_b200_rmsnorm_scatter_backward(const void* grad_normed, int64_t ld_g, const void* hidden_states, int64_t ld_x,
                                       int32_t dtype, int64_t n_rows, int64_t hidden, const void* gamma, const float* rstd,
                                       const int32_t* perm, const int32_t* active_rows, float offset, int32_t casting_mode,
                                       void* grad_hidden, int64_t ld_gx, float* grad_gamma, float* partials, void* stream_) {
  int rc = check_rmsnorm(dtype, hidden, casting_mode, gamma);
  if (rc != FLCE_OK) return rc;
  if (grad_normed == nullptr || hidden_states == nullptr || rstd == nullptr || grad_hidden == nullptr || grad_gamma == nullptr ||
      partials == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL argument");
  if (n_rows <= 0 || n_rows > 0x7fffffffll || ld_g < hidden || ld_x < hidden || ld_gx < hidden || ld_g % 8 != 0 || ld_x % 8 != 0 ||
      ld_gx % 8 != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "bad shapes (n_rows=%lld hidden=%lld pitches %lld %lld %lld)", (long long)n_rows,
                (long long)hidden, (long long)ld_g, (long long)ld_x, (long long)ld_gx);
  if (((reinterpret_cast<uintptr_t>(grad_normed) | reinterpret_cast<uintptr_t>(hidden_states) |
        reinterpret_cast<uintptr_t>(grad_hidden)) & 15) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "matrices must be 16-byte aligned");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int blocks = rmsnorm_partial_blocks();
  if (blocks > n_rows) blocks = static_cast<int>(n_rows);
  if (dtype == FLCE_BF16)
    launch_rmsnorm_backward<__nv_bfloat16>(grad_normed, ld_g, hidden_states, ld_x, gamma, rstd, perm, active_rows, n_rows, hidden,
                                           offset, casting_mode, grad_hidden, ld_gx, partials, blocks, stream);
  else
    launch_rmsnorm_backward<__half>(grad_normed, ld_g, hidden_states, ld_x, gamma, rstd, perm, active_rows, n_rows, hidden, offset,
                                    casting_mode, grad_hidden, ld_gx, partials, blocks, stream);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  rmsnorm_dgamma_reduce_kernel<<<static_cast<unsigned>(ceil_div(hidden, 256)), 256, 0, stream>>>(partials, blocks,
                                                                                               static_cast<int>(hidden), grad_gamma);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_scatter_rows(const void* src, int64_t row_bytes, const int32_t* perm, const int32_t* active_rows,
                           int64_t n_rows, void* dst, void* stream_) {
  if (src == nullptr || perm == nullptr || active_rows == nullptr || dst == nullptr || n_rows <= 0 || row_bytes <= 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "bad scatter_rows arguments");
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(src) & 15) != 0 || (reinterpret_cast<uintptr_t>(dst) & 15) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "rows must be 16-byte multiples and 16-byte aligned");
  DeviceState* dev = nullptr;
  int rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  scatter_rows_kernel<<<static_cast<unsigned>(n_rows), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(src), perm, active_rows, static_cast<uint8_t*>(dst), row_bytes);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_scale_gradient(void* data, int64_t n, int32_t dtype, const float* scale, void* stream_) {
  if (data == nullptr || scale == nullptr || n <= 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "bad scale_gradient arguments");
  if (dtype < FLCE_BF16 || dtype > FLCE_FP32) return fail(FLCE_ERR_INVALID_ARGUMENT, "bad dtype");
  DeviceState* dev = nullptr;
  int rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  const int fmt = dtype == FLCE_FP32 ? kOutFp32 : (dtype == FLCE_BF16 ? kOutBf16 : kOutFp16);
  scale_inplace_kernel<<<dev->sm_count * 8, 256, 0, static_cast<cudaStream_t>(stream_)>>>(data, n, fmt, scale);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_backward_plan(const flce_problem_t* p, size_t slab_budget_bytes, int32_t* n_slabs, int64_t* slab_cols) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (n_slabs == nullptr || slab_cols == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL output");
  const BackwardPlan plan = backward_plan(p, slab_budget_bytes, true);
  *n_slabs = plan.n_slabs;
  *slab_cols = plan.slab_cols;
  return FLCE_OK;
}

int flce_b200_forward_backward_plan(const flce_problem_t* p, size_t slab_budget_bytes, int32_t* n_chunks, int64_t* chunk_rows) {
  int rc = check_problem(p);
  if (rc != FLCE_OK) return rc;
  if (n_chunks == nullptr || chunk_rows == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL output");
  {
    DeviceState* dev = nullptr;
    (void)device_state(&dev);
  }
  const FusedPlan plan = fused_plan(p, slab_budget_bytes, true);
  *n_chunks = plan.n_chunks;
  *chunk_rows = plan.chunk_rows;
  return FLCE_OK;
}

int flce_b200_gemm(const void* a, const void* b, void* d, int64_t m, int64_t n, int64_t k, int64_t ld_a, int64_t ld_b,
                   int64_t ld_d, int32_t ab_dtype, int32_t d_dtype, int32_t a_mn_major, int32_t b_mn_major,
                   int32_t cta_pair, void* stream_) {
  if (a == nullptr || b == nullptr || d == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL matrix");
  if (ab_dtype != FLCE_BF16 && ab_dtype != FLCE_FP16) return fail(FLCE_ERR_UNSUPPORTED, "A/B must be bf16 or fp16");
  if (d_dtype != FLCE_FP32 && d_dtype != ab_dtype) return fail(FLCE_ERR_UNSUPPORTED, "D must be fp32 or the input dtype");
  if (n % 8 != 0 || ld_d % 8 != 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "n and ld_d must be multiples of 8");
  DeviceState* dev = nullptr;
  int rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  StoreEpilogue::Params ep{};
  ep.m_rows = static_cast<int>(m);
  ep.n_cols = static_cast<int>(n);
  ep.acc_in = nullptr;
  ep.acc_out = nullptr;
  ep.ld_acc = 0;
  ep.out = d;
  ep.ld_out = ld_d;
  ep.out_fmt = d_dtype == FLCE_FP32 ? kOutFp32 : (d_dtype == FLCE_BF16 ? kOutBf16 : kOutFp16);
  Operand oa{a, m, k, ld_a, a_mn_major != 0};
  Operand ob{b, n, k, ld_b, b_mn_major != 0};
  const bool pair = cta_pair != 0;
  const long long row_bytes = static_cast<long long>(kBlockM) * k * 2;
  if (!a_mn_major && !b_mn_major)
    return launch_gemm<kMajorK, kMajorK, StoreEpilogue>(*dev, kKindOther, pair, oa, ob, ab_dtype, m, n, k, row_bytes, false, ep, stream);
  if (a_mn_major && b_mn_major)
    return launch_gemm<kMajorMN, kMajorMN, StoreEpilogue>(*dev, kKindOther, pair, oa, ob, ab_dtype, m, n, k, row_bytes, true, ep, stream);
  if (!a_mn_major && b_mn_major)
    return launch_gemm<kMajorK, kMajorMN, StoreEpilogue>(*dev, kKindOther, pair, oa, ob, ab_dtype, m, n, k, row_bytes, true, ep, stream);
  return launch_gemm<kMajorMN, kMajorK, StoreEpilogue>(*dev, kKindOther, pair, oa, ob, ab_dtype, m, n, k, row_bytes, true, ep, stream);
}

int flce_b200_gemm_accumulate(const void* a, const void* b, float* acc, void* out, int64_t m, int64_t n, int64_t k,
                              int64_t ld_a, int64_t ld_b, int64_t ld_acc, int64_t ld_out, int32_t ab_dtype,
                              int32_t out_dtype, int32_t a_mn_major, int32_t b_mn_major, int32_t cta_pair, void* stream_) {
  if (a == nullptr || b == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL matrix");
  if (acc == nullptr && out == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "acc and out are both NULL");
  if (ab_dtype != FLCE_BF16 && ab_dtype != FLCE_FP16) return fail(FLCE_ERR_UNSUPPORTED, "A/B must be bf16 or fp16");
  const long long n8 = ceil_div(n, 8) * 8;
  if (out != nullptr) {
    if (out_dtype != FLCE_FP32 && out_dtype != ab_dtype) return fail(FLCE_ERR_UNSUPPORTED, "out must be fp32 or the input dtype");
    if (ld_out % 8 != 0 || ld_out < n8) return fail(FLCE_ERR_INVALID_ARGUMENT, "ld_out must be a multiple of 8 covering n");
    if ((reinterpret_cast<uintptr_t>(out) & 15) != 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "out must be 16-byte aligned");
  }
  if (acc != nullptr) {
    if (ld_acc % 4 != 0 || ld_acc < ceil_div(n, 4) * 4)
      return fail(FLCE_ERR_INVALID_ARGUMENT, "ld_acc must be a multiple of 4 covering n");
    if ((reinterpret_cast<uintptr_t>(acc) & 15) != 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "acc must be 16-byte aligned");
  }
  DeviceState* dev = nullptr;
  int rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  StoreEpilogue::Params ep{};
  ep.m_rows = static_cast<int>(m);
  ep.n_cols = static_cast<int>(n);
  ep.acc_in = acc;
  ep.acc_out = acc;
  if (acc != nullptr && out == nullptr) {
    // only the running sum is wanted: add into it at L2, nothing is read back
    ep.acc_in = nullptr;
    ep.acc_add = 1;
  }
  ep.ld_acc = ld_acc;
  ep.out = out;
  ep.ld_out = ld_out;
  ep.out_fmt = out_dtype == FLCE_FP32 ? kOutFp32 : (out_dtype == FLCE_BF16 ? kOutBf16 : kOutFp16);
  Operand oa{a, m, k, ld_a, a_mn_major != 0};
  Operand ob{b, n, k, ld_b, b_mn_major != 0};
  const bool pair = cta_pair != 0;
  const long long row_bytes = static_cast<long long>(kBlockM) * k * 2;
  if (!a_mn_major && !b_mn_major)
    return launch_gemm<kMajorK, kMajorK, StoreEpilogue>(*dev, kKindOther, pair, oa, ob, ab_dtype, m, n, k, row_bytes, false, ep, stream);
  if (a_mn_major && b_mn_major)
    return launch_gemm<kMajorMN, kMajorMN, StoreEpilogue>(*dev, kKindOther, pair, oa, ob, ab_dtype, m, n, k, row_bytes, true, ep, stream);
  if (!a_mn_major && b_mn_major)
    return launch_gemm<kMajorK, kMajorMN, StoreEpilogue>(*dev, kKindOther, pair, oa, ob, ab_dtype, m, n, k, row_bytes, true, ep, stream);
  return launch_gemm<kMajorMN, kMajorK, StoreEpilogue>(*dev, kKindOther, pair, oa, ob, ab_dtype, m, n, k, row_bytes, true, ep, stream);
}

// ------------------------------------------------------------------ chunked sibling losses: row kernels
static int check_slab(const void* slab, int64_t ld, int32_t dtype, int64_t n_rows, int64_t vocab, const char* what) {
  if (slab == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "%s is NULL", what);
  if (n_rows <= 0 || vocab <= 0 || ld < vocab)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "bad %s shape (n_rows=%lld vocab=%lld ld=%lld)", what, (long long)n_rows,
                (long long)vocab, (long long)ld);
  if (n_rows > 0x7fffffffll || vocab > 0x7fffffffll) return fail(FLCE_ERR_INVALID_ARGUMENT, "shapes must fit 32 bits");
  if (dtype < FLCE_BF16 || dtype > FLCE_FP32) return fail(FLCE_ERR_UNSUPPORTED, "%s must be bf16, fp16 or fp32", what);
  return FLCE_OK;
}

int flce_b200_scaled_ce_rows(const void* logits, int64_t ld, int32_t dtype, int64_t n_rows, int64_t vocab,
                             const int64_t* target_, int64_t ignore_index, float temperature, float* nll, float* entropy,
                             float* lse, void* stream_) {
  int rc = check_slab(logits, ld, dtype, n_rows, vocab, "logits");
  if (rc != FLCE_OK) return rc;
  if (target_ == nullptr || nll == nullptr || entropy == nullptr || lse == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "target, nll, entropy and lse must not be NULL");
  if (!(temperature > 0.f) || !isfinite(temperature)) return fail(FLCE_ERR_INVALID_ARGUMENT, "temperature must be finite and > 0");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long* target = reinterpret_cast<const long long*>(target_);
  const float inv_t = 1.f / temperature;
  if (dtype == FLCE_FP32) launch_scaled_ce_rows<float>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, nll, entropy, lse, stream);
  else if (dtype == FLCE_BF16) launch_scaled_ce_rows<__nv_bfloat16>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, nll, entropy, lse, stream);
  else launch_scaled_ce_rows<__half>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, nll, entropy, lse, stream);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_scaled_ce_grad(void* logits, int64_t ld, int32_t dtype, int64_t n_rows, int64_t vocab, const int64_t* target_,
                             int64_t ignore_index, float temperature, const float* lse, const float* entropy,
                             const float* grad_nll, const float* grad_entropy, void* stream_) {
  int rc = check_slab(logits, ld, dtype, n_rows, vocab, "logits");
  if (rc != FLCE_OK) return rc;
  if (target_ == nullptr || lse == nullptr || entropy == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "target, lse and entropy must not be NULL");
  if (!(temperature > 0.f) || !isfinite(temperature)) return fail(FLCE_ERR_INVALID_ARGUMENT, "temperature must be finite and > 0");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long* target = reinterpret_cast<const long long*>(target_);
  const float inv_t = 1.f / temperature;
  if (dtype == FLCE_FP32) launch_scaled_ce_grad<float>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, lse, entropy, grad_nll, grad_entropy, stream);
  else if (dtype == FLCE_BF16) launch_scaled_ce_grad<__nv_bfloat16>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, lse, entropy, grad_nll, grad_entropy, stream);
  else launch_scaled_ce_grad<__half>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, lse, entropy, grad_nll, grad_entropy, stream);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_jsd_rows(void* student, int64_t ld_student, const void* teacher, int64_t ld_teacher, int32_t dtype,
                       int64_t n_rows, int64_t vocab, const int64_t* labels_, int64_t ignore_index, float beta,
                       float temperature, const float* count, float fixed_count, float* loss_rows, void* stream_) {
  int rc = check_slab(student, ld_student, dtype, n_rows, vocab, "student logits");
  if (rc != FLCE_OK) return rc;
  rc = check_slab(teacher, ld_teacher, dtype, n_rows, vocab, "teacher logits");
  if (rc != FLCE_OK) return rc;
  if (loss_rows == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "loss_rows must not be NULL");
  if (!(beta >= 0.f && beta <= 1.f)) return fail(FLCE_ERR_INVALID_ARGUMENT, "beta must be in [0, 1]");
  if (temperature == 0.f || !isfinite(temperature)) return fail(FLCE_ERR_INVALID_ARGUMENT, "temperature must be finite and not 0");
  if (count == nullptr && !(fixed_count > 0.f)) return fail(FLCE_ERR_INVALID_ARGUMENT, "fixed_count must be positive when count is NULL");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long* labels = reinterpret_cast<const long long*>(labels_);
  const float inv_t = 1.f / temperature;
  if (dtype == FLCE_FP32) launch_jsd_rows<float>(dev->sm_count, student, ld_student, teacher, ld_teacher, dtype, n_rows, vocab, labels, ignore_index, beta, inv_t, count, fixed_count, loss_rows, stream);
  else if (dtype == FLCE_BF16) launch_jsd_rows<__nv_bfloat16>(dev->sm_count, student, ld_student, teacher, ld_teacher, dtype, n_rows, vocab, labels, ignore_index, beta, inv_t, count, fixed_count, loss_rows, stream);
  else launch_jsd_rows<__half>(dev->sm_count, student, ld_student, teacher, ld_teacher, dtype, n_rows, vocab, labels, ignore_index, beta, inv_t, count, fixed_count, loss_rows, stream);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

// ------------------------------------------------------------------ scaled cross-entropy on the two sweeps
static int sce_as_problem(const flce_sce_problem_t* p, flce_problem_t* q) {
  if (p == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "problem is NULL");
  if (!(p->temperature > 0.f) || !isfinite(p->temperature))
    return fail(FLCE_ERR_INVALID_ARGUMENT, "temperature must be finite and > 0");
  memset(q, 0, sizeof(*q));
  q->n_rows = p->n_rows;
  q->hidden = p->hidden;
  q->vocab = p->vocab;
  q->vocab_total = p->vocab;
  q->vocab_offset = 0;
  q->ld_x = p->ld_x;
  q->ld_w = p->ld_w;
  q->dtype = p->dtype;
  q->reduction = FLCE_NONE;
  q->ignore_index = p->ignore_index;
  q->x = p->x;
  q->w = p->w;
  q->target = p->target;
  return check_problem(q);   // shapes, pitches, alignment, dtype: the same rules as the main path
}

struct ScePlan {
  int n_tiles;
  size_t plane;   // bytes of one [n_tiles][n_rows] fp32 plane
  size_t target_logit_bytes;
  size_t total;
};
static ScePlan sce_forward_plan(const flce_problem_t* q) {
  ScePlan f;
  f.n_tiles = static_cast<int>(ceil_div(q->vocab, kBlockN));
  f.plane = align_up(static_cast<size_t>(f.n_tiles) * q->n_rows * sizeof(float), 256);
  f.target_logit_bytes = align_up(static_cast<size_t>(q->n_rows) * sizeof(float), 256);
  f.total = 3 * f.plane + f.target_logit_bytes;
  return f;
}

size_t flce_b200_sce_workspace_bytes(const flce_sce_problem_t* p, int phase, size_t slab_budget_bytes) {
  flce_problem_t q;
  if (sce_as_problem(p, &q) != FLCE_OK) return 0;
  if (phase == FLCE_PHASE_FORWARD) return sce_forward_plan(&q).total;
  if (phase == FLCE_PHASE_BACKWARD) {
    const BackwardPlan b = backward_plan(&q, slab_budget_bytes, true);
    return b.slab_bytes + b.acc_bytes;
  }
  return 0;
}

int flce_b200_sce_forward(const flce_sce_problem_t* p, float* nll, float* entropy, float* lse, void* workspace,
                          size_t workspace_bytes, void* stream_) {
  flce_problem_t q;
  int rc = sce_as_problem(p, &q);
  if (rc != FLCE_OK) return rc;
  if (nll == nullptr || entropy == nullptr || lse == nullptr)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "nll, entropy and lse must not be NULL");
  const ScePlan plan = sce_forward_plan(&q);
  if (workspace == nullptr || workspace_bytes < plan.total)
    return fail(FLCE_ERR_WORKSPACE, "scaled cross-entropy forward needs %zu bytes of workspace, got %zu", plan.total,
                workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  EntropyStatsEpilogue::Params ep{};
  ep.target = reinterpret_cast<const long long*>(p->target);
  ep.scale = 1.f / p->temperature;
  ep.n_cols = static_cast<int>(p->vocab);
  ep.m_rows = static_cast<int>(p->n_rows);
  ep.pmax = reinterpret_cast<float*>(ws);
  ep.psum = reinterpret_cast<float*>(ws + plan.plane);
  ep.pts = reinterpret_cast<float*>(ws + 2 * plan.plane);
  ep.target_logit = reinterpret_cast<float*>(ws + 3 * plan.plane);
  FLCE_CUDA(cudaMemsetAsync(ep.target_logit, 0, static_cast<size_t>(p->n_rows) * sizeof(float), stream));
  Operand a{p->x, p->n_rows, p->hidden, p->ld_x, 0};
  Operand b{p->w, p->vocab, p->hidden, p->ld_w, 0};
  rc = launch_gemm<kMajorK, kMajorK, EntropyStatsEpilogue>(*dev, kKindStats, g_cta_pair != 0, a, b, p->dtype, p->n_rows, p->vocab,
                                                           p->hidden, static_cast<long long>(kBlockM) * p->hidden * 2, false, ep,
                                                           stream);
  if (rc != FLCE_OK) return rc;
  const int threads = 256;
  scaled_ce_merge_kernel<<<static_cast<unsigned>(ceil_div(p->n_rows, threads)), threads, 0, stream>>>(
      static_cast<int>(p->n_rows), plan.n_tiles, ep.pmax, ep.psum, ep.pts, ep.target_logit,
      reinterpret_cast<const long long*>(p->target), p->ignore_index, nll, entropy, lse);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_sce_backward(const flce_sce_problem_t* p, const float* lse, const float* entropy, const float* grad_nll,
                           const float* grad_entropy, int32_t grad_dtype, void* grad_input, void* grad_weight,
                           void* workspace, size_t workspace_bytes, size_t slab_budget_bytes, void* stream_) {
  flce_problem_t q;
  int rc = sce_as_problem(p, &q);
  if (rc != FLCE_OK) return rc;
  if (lse == nullptr || entropy == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "lse and entropy must not be NULL");
  if (grad_dtype != p->dtype && grad_dtype != FLCE_FP32)
    return fail(FLCE_ERR_UNSUPPORTED, "gradients must be in the input dtype or fp32");
  if (p->hidden % 8 != 0) return fail(FLCE_ERR_INVALID_ARGUMENT, "hidden must be a multiple of 8 (pad the operands)");
  const bool grads_fp32 = grad_dtype == FLCE_FP32;
  const BackwardPlan plan = backward_plan(&q, slab_budget_bytes, true);
  const size_t needed = plan.slab_bytes + ((grad_input != nullptr && !grads_fp32) ? plan.acc_bytes : 0);
  if (workspace == nullptr || workspace_bytes < needed)
    return fail(FLCE_ERR_WORKSPACE, "scaled cross-entropy backward needs %zu bytes of workspace, got %zu", needed,
                workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
  DeviceState* dev = nullptr;
  rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint16_t* dz = reinterpret_cast<uint16_t*>(ws);
  float* dx_acc = reinterpret_cast<float*>(ws + plan.slab_bytes);   // unused with fp32 gradients
  const bool pair = g_cta_pair != 0;
  const int esize_out = grads_fp32 ? 4 : 2;
  const int fmt16 = p->dtype == FLCE_BF16 ? kOutBf16 : kOutFp16;
  for (int s = 0; s < plan.n_slabs; ++s) {
    const long long v0 = static_cast<long long>(s) * plan.slab_cols;
    const long long cols = (p->vocab - v0 < plan.slab_cols) ? p->vocab - v0 : plan.slab_cols;
    const uint16_t* w_slab = static_cast<const uint16_t*>(p->w) + v0 * p->ld_w;
    {  // recompute the logits of this slab -> dZ
      ScaledDzEpilogue::Params ep;
      ep.target = reinterpret_cast<const long long*>(p->target);
      ep.ignore_index = p->ignore_index;
      ep.scale = 1.f / p->temperature;
      ep.n_cols = static_cast<int>(cols);
      ep.vocab_offset = v0;
      ep.m_rows = static_cast<int>(p->n_rows);
      ep.lse = lse;
      ep.entropy = entropy;
      ep.grad_nll = grad_nll;
      ep.grad_entropy = grad_entropy;
      ep.dz = dz;
      ep.ld_dz = plan.ld_dz;
      ep.out_fmt = fmt16;
      Operand a{p->x, p->n_rows, p->hidden, p->ld_x, 0};
      Operand b{w_slab, cols, p->hidden, p->ld_w, 0};
      rc = launch_gemm<kMajorK, kMajorK, ScaledDzEpilogue>(*dev, kKindDz, pair, a, b, p->dtype, p->n_rows, cols, p->hidden,
                                                           static_cast<long long>(kBlockM) * p->hidden * 2, false, ep, stream);
      if (rc != FLCE_OK) return rc;
    }
    if (grad_weight != nullptr) {  // grad_weight[slab] = dZ^T . X   (M = cols, N = hidden, K = n_rows; both MN-major)
      StoreEpilogue::Params ep{};
      ep.m_rows = static_cast<int>(cols);
      ep.n_cols = static_cast<int>(p->hidden);
      ep.acc_in = nullptr;
      ep.acc_out = nullptr;
      ep.ld_acc = 0;
      ep.out = static_cast<uint8_t*>(grad_weight) + static_cast<size_t>(v0) * p->hidden * esize_out;
      ep.ld_out = p->hidden;
      ep.out_fmt = grads_fp32 ? kOutFp32 : fmt16;
      Operand a{dz, cols, p->n_rows, plan.ld_dz, 1};
      Operand b{p->x, p->hidden, p->n_rows, p->ld_x, 1};
      rc = launch_gemm<kMajorMN, kMajorMN, StoreEpilogue>(*dev, kKindDw, pair, a, b, p->dtype, cols, p->hidden, p->n_rows, 0, true,
                                                          ep, stream);
      if (rc != FLCE_OK) return rc;
    }
    if (grad_input != nullptr) {  // grad_input (+)= dZ . W[slab]   (M = n_rows, N = hidden, K = cols; B MN-major)
      StoreEpilogue::Params ep{};
      ep.m_rows = static_cast<int>(p->n_rows);
      ep.n_cols = static_cast<int>(p->hidden);
      const bool first = s == 0, last = s == plan.n_slabs - 1;
      float* acc = grads_fp32 ? static_cast<float*>(grad_input) : dx_acc;
      ep.acc_in = first ? nullptr : acc;
      ep.acc_out = (last && !grads_fp32) ? nullptr : acc;
      if (plan.n_slabs == 1 && !grads_fp32) ep.acc_out = nullptr;
      ep.ld_acc = p->hidden;
      ep.out = (last && !grads_fp32) ? grad_input : nullptr;
      ep.ld_out = p->hidden;
      ep.out_fmt = fmt16;
      Operand a{dz, p->n_rows, cols, plan.ld_dz, 0};
      Operand b{w_slab, p->hidden, cols, p->ld_w, 1};
      rc = launch_gemm<kMajorK, kMajorMN, StoreEpilogue>(*dev, kKindDx, pair, a, b, p->dtype, p->n_rows, p->hidden, cols, 0, true,
                                                         ep, stream);
      if (rc != FLCE_OK) return rc;
    }
  }
  return FLCE_OK;
}

int flce_b200_profile_enable(int on) {
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  g_profile_on = on != 0;
  g_profile_used = 0;
  return FLCE_OK;
}

int flce_b200_profile_read(double* ms_by_kind, int64_t* launches_by_kind, int reset) {
  if (ms_by_kind == nullptr || launches_by_kind == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "NULL output");
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  for (int k = 0; k < kNumKinds; ++k) {
    ms_by_kind[k] = 0.0;
    launches_by_kind[k] = 0;
  }
  for (int i = 0; i < g_profile_used; ++i) {
    FLCE_CUDA(cudaEventSynchronize(g_profile[i].stop));
    float ms = 0.f;
    FLCE_CUDA(cudaEventElapsedTime(&ms, g_profile[i].start, g_profile[i].stop));
    ms_by_kind[g_profile[i].kind] += ms;
    launches_by_kind[g_profile[i].kind] += 1;
  }
  if (reset) g_profile_used = 0;
  return FLCE_OK;
}

int64_t flce_b200_kernel_launches(void) { return g_kernel_launches; }

#ifdef FLCE_CLOCK_TRACE
int flce_b200_debug_clock_trace(unsigned long long* out, int n_words) {
  FLCE_CUDA(cudaDeviceSynchronize());
  FLCE_CUDA(cudaMemcpyFromSymbol(out, g_clock_trace, sizeof(unsigned long long) * n_words));
  return FLCE_OK;
}
#endif

int flce_b200_selftest_wait_expiry(int64_t limit_ns, int32_t* outcome, void* stream_) {
  if (limit_ns <= 0 || limit_ns > 100000000ll)
    return fail(FLCE_ERR_INVALID_ARGUMENT, "limit_ns must be in (0, 1e8] (at most a tenth of a second)");
  if (outcome == nullptr) return fail(FLCE_ERR_INVALID_ARGUMENT, "outcome is NULL");
  DeviceState* dev = nullptr;
  int rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  FLCE_CUDA(cudaMemsetAsync(outcome, 0, sizeof(int32_t), stream));
  wait_expiry_selftest_kernel<<<1, 32, 0, stream>>>(static_cast<unsigned long long>(limit_ns), dev->status, outcome);
  FLCE_CUDA(cudaGetLastError());
  ++g_kernel_launches;
  return FLCE_OK;
}

int flce_b200_check_device_status(void* stream) {
  DeviceState* dev = nullptr;
  int rc = device_state(&dev);
  if (rc != FLCE_OK) return rc;
  FLCE_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int word = 0;
  FLCE_CUDA(cudaMemcpy(&word, dev->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (word != 0) {
    FLCE_CUDA(cudaMemset(dev->status, 0, sizeof(int)));
    return fail(FLCE_ERR_DEVICE_TIMEOUT, "a kernel abandoned a bounded wait (device status %d)", word);
  }
  return FLCE_OK;
}

}  // extern "C"
