// The library's SIMT kernels (csrc/row_kernels.cuh, csrc/ce_kernels.cuh, csrc/head_loss_kernels.cuh), the register
// epilogues of its tensor-core sweeps (csrc/epilogues.cuh) and its tile schedule (csrc/tile_schedule.cuh) compiled for the host and run on the host
// through simt_emulation.hpp, behind a small C interface for the CPU tests.  Every wrapper repeats the launch geometry
// and kernel order of the library entry point it is named after (csrc/flce_b200.cu), so the tests exercise the same
// index arithmetic a GPU launch would.  ex2.approx / rcp.approx are replaced by libm (FLCE_HOST_EMULATION), so results
// agree with the GPU to a few ulp, not bit for bit.
//
// Test infrastructure only.
#define FLCE_HOST_EMULATION 1
#define FLCE_JSD_THREADS 256   // 1024 on the GPU; fewer fibers keep the emulated barriers cheap, the code is the same
#include "simt_emulation.hpp"

#include "ce_kernels.cuh"
#include "epilogues.cuh"
#include "head_loss_kernels.cuh"
#include "rmsnorm_rows.cuh"
#include "row_kernels.cuh"
#include "tile_schedule.cuh"

using namespace flce;

namespace {

long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

struct CeProblem {
  int dtype;  // 0 bf16, 1 fp16, 2 fp32
  const void* logits;
  long long ld, n_rows, vocab;
  const long long* target;
  const float* ce_weight;
  long long ignore_index;
  float label_smoothing, lse_square_scale, softcap;
  int reduction;  // 0 mean, 1 sum, 2 none
};

RowMath row_math(const CeProblem& p) {
  RowMath rm;
  rm.ignore_index = p.ignore_index;
  rm.alpha = p.label_smoothing;
  rm.eps = p.label_smoothing / static_cast<float>(p.vocab);
  rm.lambda = p.lse_square_scale;
  rm.mean = p.reduction == 0;
  rm.token_scaling = 0;
  rm.weighted = p.ce_weight != nullptr;
  rm.vocab = p.vocab;
  rm.vocab_offset = 0;
  return rm;
}

bool vectorisable(const void* base, long long ld, int dtype) {
  const long long esize = dtype == 2 ? 4 : 2;
  return (reinterpret_cast<uintptr_t>(base) & 15) == 0 && (ld * esize) % 16 == 0;
}

template <typename T>
void run_ce_stats(const CeProblem& p, float* rowstats) {
  const float inv = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
  const T* x = static_cast<const T*>(p.logits);
  const bool vec = vectorisable(p.logits, p.ld, p.dtype);
  emu::launch(emu::Dim3(static_cast<unsigned>(p.n_rows)), emu::Dim3(kCeThreads), [&]() {
    if (vec)
      ce_stats_kernel<T, true>(x, p.ld, static_cast<int>(p.n_rows), static_cast<int>(p.vocab), p.target, p.ce_weight,
                               p.softcap, inv, rowstats);
    else
      ce_stats_kernel<T, false>(x, p.ld, static_cast<int>(p.n_rows), static_cast<int>(p.vocab), p.target, p.ce_weight,
                                p.softcap, inv, rowstats);
  });
}

template <typename T>
void run_ce_grad(const CeProblem& p, void* grad, long long ld_grad, const float* lse, const float* c1, const float* c2,
                 const float* c3) {
  const float inv = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
  const T* x = static_cast<const T*>(p.logits);
  const bool vec = vectorisable(p.logits, p.ld, p.dtype) && vectorisable(grad, ld_grad, p.dtype);
  const long long per_thread = vec ? CeElem<T>::kVec : 1;
  const emu::Dim3 grid(static_cast<unsigned>(p.n_rows),
                       static_cast<unsigned>(ceil_div(ceil_div(p.vocab, per_thread), kCeThreads * kCeGradUnroll)), 1);
  emu::launch_serial(grid, emu::Dim3(kCeThreads), [&]() {
    if (vec)
      ce_grad_kernel<T, true>(x, p.ld, static_cast<T*>(grad), ld_grad, static_cast<int>(p.n_rows),
                              static_cast<int>(p.vocab), p.target, p.ce_weight, p.softcap, inv, lse, c1, c2, c3);
    else
      ce_grad_kernel<T, false>(x, p.ld, static_cast<T*>(grad), ld_grad, static_cast<int>(p.n_rows),
                               static_cast<int>(p.vocab), p.target, p.ce_weight, p.softcap, inv, lse, c1, c2, c3);
  });
}

CeProblem make_problem(int dtype, const void* logits, long long ld, long long n_rows, long long vocab,
                       const long long* target, const float* ce_weight, long long ignore_index, float label_smoothing,
                       float lse_square_scale, float softcap, int reduction) {
  CeProblem p;
  p.dtype = dtype;
  p.logits = logits;
  p.ld = ld;
  p.n_rows = n_rows;
  p.vocab = vocab;
  p.target = target;
  p.ce_weight = ce_weight;
  p.ignore_index = ignore_index;
  p.label_smoothing = label_smoothing;
  p.lse_square_scale = lse_square_scale;
  p.softcap = softcap;
  p.reduction = reduction;
  return p;
}

template <typename T>
void run_scaled_ce_rows(const void* logits, long long ld, int dtype, long long n_rows, long long vocab, const long long* target,
                        long long ignore_index, float inv_t, float* nll, float* entropy, float* lse) {
  const T* x = static_cast<const T*>(logits);
  const bool vec = vectorisable(logits, ld, dtype);
  emu::launch(emu::Dim3(static_cast<unsigned>(n_rows)), emu::Dim3(kCeThreads), [&]() {
    if (vec)
      scaled_ce_rows_kernel<T, true>(x, ld, static_cast<int>(n_rows), static_cast<int>(vocab), target, ignore_index, inv_t, nll,
                                     entropy, lse);
    else
      scaled_ce_rows_kernel<T, false>(x, ld, static_cast<int>(n_rows), static_cast<int>(vocab), target, ignore_index, inv_t, nll,
                                      entropy, lse);
  });
}

template <typename T>
void run_scaled_ce_grad(void* logits, long long ld, int dtype, long long n_rows, long long vocab, const long long* target,
                        long long ignore_index, float inv_t, const float* lse, const float* entropy, const float* g_nll,
                        const float* g_ent) {
  const bool vec = vectorisable(logits, ld, dtype);
  const long long per_thread = vec ? CeElem<T>::kVec : 1;
  const emu::Dim3 grid(static_cast<unsigned>(n_rows), static_cast<unsigned>(ceil_div(ceil_div(vocab, per_thread), kCeThreads)), 1);
  T* x = static_cast<T*>(logits);
  emu::launch_serial(grid, emu::Dim3(kCeThreads), [&]() {
    if (vec)
      scaled_ce_grad_kernel<T, true>(x, ld, static_cast<int>(n_rows), static_cast<int>(vocab), target, ignore_index, inv_t, lse,
                                     entropy, g_nll, g_ent);
    else
      scaled_ce_grad_kernel<T, false>(x, ld, static_cast<int>(n_rows), static_cast<int>(vocab), target, ignore_index, inv_t, lse,
                                      entropy, g_nll, g_ent);
  });
}

template <typename T>
void run_jsd_rows(void* student, long long ld_s, const void* teacher, long long ld_t, int dtype, long long n_rows, long long vocab,
                  const long long* labels, long long ignore_index, float beta, float inv_t, const float* count,
                  float fixed_count, float* loss_rows) {
  const bool vec = vectorisable(student, ld_s, dtype) && vectorisable(teacher, ld_t, dtype);
  T* xs = static_cast<T*>(student);
  const T* xt = static_cast<const T*>(teacher);
  const unsigned grid = static_cast<unsigned>(std::min<long long>(n_rows, 148));   // one CTA per SM walks over the rows
  emu::launch(emu::Dim3(grid), emu::Dim3(kJsdThreads), [&]() {
    if (vec)
      jsd_rows_kernel<T, true>(xs, ld_s, xt, ld_t, static_cast<int>(n_rows), static_cast<int>(vocab), labels, ignore_index, beta,
                               inv_t, count, fixed_count, loss_rows);
    else
      jsd_rows_kernel<T, false>(xs, ld_s, xt, ld_t, static_cast<int>(n_rows), static_cast<int>(vocab), labels, ignore_index, beta,
                                inv_t, count, fixed_count, loss_rows);
  });
}

// ---- the tensor-core sweeps at tile level: the main loop's accumulators are replaced by a float dot product of the 16-bit
// operands (what the tensor cores compute up to summation order, zeros where TMA would fill out-of-range rows / columns), and
// each epilogue instance is driven the way an epilogue thread of gemm_tcgen05_kernel drives it: begin, up to eight chunks of
// 32 accumulators, end -- for every row of every 128 x 256 tile, including the rows of the last tile that lie beyond M.
float load16(const void* base, long long index, int dtype) {
  if (dtype == 0) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[index]);
  return __half2float(static_cast<const __half*>(base)[index]);
}

template <class Epi>
void run_tiles(const typename Epi::Params& ep, const void* a, const void* b, int dtype, int m, int n, int k, long long ld_a,
               long long ld_b, int m_tile_limit = -1) {
  int m_tiles = static_cast<int>(ceil_div(m, kBlockM));
  if (m_tile_limit >= 0) m_tiles = std::min(m_tiles, m_tile_limit);   // tiles a device-resident active-row count leaves
  const int n_tiles = static_cast<int>(ceil_div(n, kBlockN));
  std::vector<float> arow(k);
  for (int mt = 0; mt < m_tiles; ++mt)
    for (int r = 0; r < kBlockM; ++r) {
      const int row = mt * kBlockM + r;
      const bool ok = row < m;
      for (int kk = 0; kk < k; ++kk) arow[kk] = ok ? load16(a, static_cast<long long>(row) * ld_a + kk, dtype) : 0.f;
      for (int nt = 0; nt < n_tiles; ++nt) {
        const int col0 = nt * kBlockN;
        Epi epi;
        epi.begin(ep, row, col0, nt, ok);
        const int n_chunks = std::min(kBlockN / 32, (n - col0 + 31) / 32);
        for (int c = 0; c < n_chunks; ++c) {
          uint32_t acc[32];
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + c * 32 + j;
            float v = 0.f;
            if (ok && col < n)
              for (int kk = 0; kk < k; ++kk) v = fmaf(arow[kk], load16(b, static_cast<long long>(col) * ld_b + kk, dtype), v);
            acc[j] = __float_as_uint(v);
          }
          epi.chunk(ep, acc, col0 + c * 32, nullptr, nullptr);
        }
        epi.end(ep);
      }
    }
}

// StoreEpilogue passes its accumulators through a warp-wide shared-memory patch, so its 32 rows run together: one
// emulated warp per group of 32 rows, driven over the n-tiles the way an epilogue warp of the kernel is.
void run_tiles_store(const StoreEpilogue::Params& ep, const void* a, const void* b, int dtype, int m, int n, int k, long long ld_a,
                     long long ld_b, int tile_n) {
  const int groups = static_cast<int>(ceil_div(m, kBlockM)) * (kBlockM / 32);
  const int n_tiles = static_cast<int>(ceil_div(n, tile_n));
  static float stage[2048];
  for (int g = 0; g < groups; ++g) {
    emu::launch(1, 32, [&]() {
      const int lane = static_cast<int>(threadIdx.x);
      const int row = g * 32 + lane;
      const bool ok = row < m;
      std::vector<float> arow(k);
      for (int kk = 0; kk < k; ++kk) arow[kk] = ok ? load16(a, static_cast<long long>(row) * ld_a + kk, dtype) : 0.f;
      for (int nt = 0; nt < n_tiles; ++nt) {
        const int col0 = nt * tile_n;
        StoreEpilogue epi;
        epi.begin(ep, row, col0, nt, ok);
        const int n_chunks = std::min(tile_n / 32, (n - col0 + 31) / 32);
        for (int c = 0; c < n_chunks; ++c) {
          uint32_t acc[32];
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + c * 32 + j;
            float v = 0.f;
            if (ok && col < n)
              for (int kk = 0; kk < k; ++kk) v = fmaf(arow[kk], load16(b, static_cast<long long>(col) * ld_b + kk, dtype), v);
            acc[j] = __float_as_uint(v);
          }
          epi.chunk(ep, acc, col0 + c * 32, stage, nullptr);
        }
        epi.end(ep);
      }
    });
  }
}

}  // namespace

extern "C" {

// the kernel sequence of flce_b200_ce_forward; any of the per-row outputs and scalars may be null
int emu_ce_forward(int dtype, const void* logits, long long ld, long long n_rows, long long vocab, const long long* target,
                   const float* ce_weight, long long ignore_index, float label_smoothing, float lse_square_scale,
                   float softcap, int reduction, float* norm, float* rowstats, float* lse, float* target_prob,
                   float* loss_rows, float* z_rows, float* correct_rows, long long* predicted, float* scalars) {
  const CeProblem p = make_problem(dtype, logits, ld, n_rows, vocab, target, ce_weight, ignore_index, label_smoothing,
                                   lse_square_scale, softcap, reduction);
  emu::launch(1, kRedThreads, [&]() {
    count_kernel(target, n_rows, ignore_index, ce_weight, vocab, 0, static_cast<float>(vocab), norm);
  });
  if (dtype == 2) run_ce_stats<float>(p, rowstats);
  else if (dtype == 0) run_ce_stats<__nv_bfloat16>(p, rowstats);
  else run_ce_stats<__half>(p, rowstats);
  const int threads = 256;
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_rows, threads)), threads, [&]() {
    finalize_rows_kernel(static_cast<int>(n_rows), row_math(p), target, ce_weight, rowstats, norm, lse, target_prob,
                         loss_rows, z_rows, correct_rows, predicted);
  });
  if (scalars != nullptr)
    emu::launch(1, kRedThreads, [&]() {
      reduce_rows_kernel(static_cast<int>(n_rows), loss_rows, z_rows, correct_rows, norm, scalars);
    });
  return 0;
}

// the kernel sequence of flce_b200_ce_backward; grad may alias logits
int emu_ce_backward(int dtype, const void* logits, long long ld, long long n_rows, long long vocab, const long long* target,
                    const float* ce_weight, long long ignore_index, float label_smoothing, float lse_square_scale,
                    float softcap, int reduction, const float* lse, const float* norm, const float* grad_output,
                    int per_row, void* grad, long long ld_grad, float* coef_scratch) {
  const CeProblem p = make_problem(dtype, logits, ld, n_rows, vocab, target, ce_weight, ignore_index, label_smoothing,
                                   lse_square_scale, softcap, reduction);
  float* c1 = coef_scratch;
  float* c2 = c1 + n_rows;
  float* c3 = c2 + n_rows;
  const int threads = 256;
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_rows, threads)), threads, [&]() {
    coef_kernel(static_cast<int>(n_rows), row_math(p), target, ce_weight, lse, nullptr, norm, grad_output, per_row, c1, c2,
                c3);
  });
  if (dtype == 2) run_ce_grad<float>(p, grad, ld_grad, lse, c1, c2, c3);
  else if (dtype == 0) run_ce_grad<__nv_bfloat16>(p, grad, ld_grad, lse, c1, c2, c3);
  else run_ce_grad<__half>(p, grad, ld_grad, lse, c1, c2, c3);
  return 0;
}

// flce_b200_count
int emu_count(const long long* target, long long n_rows, long long ignore_index, const float* ce_weight, long long vocab,
              long long vocab_offset, float vocab_total, float* norm) {
  emu::launch(1, kRedThreads, [&]() {
    count_kernel(target, n_rows, ignore_index, ce_weight, vocab, vocab_offset, vocab_total, norm);
  });
  return 0;
}

// flce_b200_compact_rows (16-bit rows of `hidden` elements, source pitch ld_x elements)
int emu_compact_rows(const void* x, long long ld_x, long long hidden, long long n_rows, const long long* target,
                     long long ignore_index, void* x_compact, long long* target_compact, int* perm, int* active) {
  emu::launch(1, kRedThreads, [&]() { compact_plan_kernel(target, static_cast<int>(n_rows), ignore_index, perm, active); });
  emu::launch_serial(static_cast<unsigned>(n_rows), 256, [&]() {
    gather_rows_kernel(static_cast<const uint8_t*>(x), ld_x * 2, perm, static_cast<uint8_t*>(x_compact), hidden * 2, target,
                       target_compact);
  });
  return 0;
}

// flce_b200_compact_rows_rmsnorm (dtype: 0 bf16, 1 fp16)
int emu_compact_rows_rmsnorm(const void* x, long long ld_x, long long hidden, long long n_rows, const long long* target,
                             long long ignore_index, int dtype, const void* gamma, float eps, float offset, int mode,
                             void* x_compact, long long* target_compact, int* perm, int* active, float* rstd) {
  emu::launch(1, kRedThreads, [&]() { compact_plan_kernel(target, static_cast<int>(n_rows), ignore_index, perm, active); });
  emu::launch(static_cast<unsigned>(n_rows), kRmsThreads, [&]() {
    if (dtype == 0)
      rmsnorm_gather_rows_kernel<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(x), ld_x, perm,
                                                static_cast<__nv_bfloat16*>(x_compact), hidden, static_cast<int>(hidden),
                                                static_cast<const __nv_bfloat16*>(gamma), eps, offset, mode, rstd, target,
                                                target_compact);
    else
      rmsnorm_gather_rows_kernel<__half>(static_cast<const __half*>(x), ld_x, perm, static_cast<__half*>(x_compact), hidden,
                                         static_cast<int>(hidden), static_cast<const __half*>(gamma), eps, offset, mode, rstd,
                                         target, target_compact);
  });
  return 0;
}

// flce_b200_rmsnorm_scatter_backward with `blocks` row-striding blocks of 256 threads (hidden <= 8192)
int emu_rmsnorm_scatter_backward(const void* gy, long long ld_g, const void* x, long long ld_x, int dtype, long long n_rows,
                                 long long hidden, const void* gamma, const float* rstd, const int* perm, const int* active,
                                 float offset, int mode, void* gx, long long ld_gx, float* dgamma, float* partials, int blocks) {
  if (hidden > 256 * 4 * 8) return 2;
  emu::launch(static_cast<unsigned>(blocks), 256, [&]() {
    if (dtype == 0)
      rmsnorm_backward_scatter_kernel<__nv_bfloat16, 4>(
          static_cast<const __nv_bfloat16*>(gy), ld_g, static_cast<const __nv_bfloat16*>(x), ld_x,
          static_cast<const __nv_bfloat16*>(gamma), rstd, perm, active, static_cast<int>(n_rows), static_cast<int>(hidden), offset,
          mode, static_cast<__nv_bfloat16*>(gx), ld_gx, partials);
    else
      rmsnorm_backward_scatter_kernel<__half, 4>(static_cast<const __half*>(gy), ld_g, static_cast<const __half*>(x), ld_x,
                                                 static_cast<const __half*>(gamma), rstd, perm, active, static_cast<int>(n_rows),
                                                 static_cast<int>(hidden), offset, mode, static_cast<__half*>(gx), ld_gx, partials);
  });
  emu::launch_serial(static_cast<unsigned>((hidden + 255) / 256), 256,
                     [&]() { rmsnorm_dgamma_reduce_kernel(partials, blocks, static_cast<int>(hidden), dgamma); });
  return 0;
}

// flce_b200_scatter_rows
int emu_scatter_rows(const void* src, long long row_bytes, const int* perm, const int* active, long long n_rows, void* dst) {
  emu::launch_serial(static_cast<unsigned>(n_rows), 256, [&]() {
    scatter_rows_kernel(static_cast<const uint8_t*>(src), perm, active, static_cast<uint8_t*>(dst), row_bytes);
  });
  return 0;
}

// flce_b200_split_fp32
int emu_split_fp32(const float* src, long long rows, long long cols, long long ld_src, void* dst, long long ld_dst,
                   long long block_cols, const int* pattern, int n_blocks, int dst_dtype) {
  SplitPattern pat;
  for (int b = 0; b < 8; ++b) pat.term[b] = b < n_blocks ? pattern[b] : 0;
  const emu::Dim3 grid(static_cast<unsigned>(ceil_div(block_cols, 256)), static_cast<unsigned>(rows), 1);
  emu::launch_serial(grid, 256, [&]() {
    split_fp32_kernel(src, rows, cols, ld_src, static_cast<uint16_t*>(dst), ld_dst, block_cols, pat, n_blocks,
                      dst_dtype == 0 ? kOutBf16 : kOutFp16);
  });
  return 0;
}

// the single-sweep mode's in-place logit gradient over one token chunk (launch geometry of flce_b200_forward_backward)
int emu_dz_inplace(void* slab, long long ld, long long rows, long long vocab, int fmt, const long long* target,
                   long long vocab_offset, const float* lse, const float* c1, const float* c2, const float* c3,
                   const float* col_weight, float inv_softcap, const int* active_rows, int active_base) {
  const emu::Dim3 grid(static_cast<unsigned>(ceil_div(vocab, kDzInplaceCols)), static_cast<unsigned>(rows), 1);
  emu::launch_serial(grid, kDzInplaceThreads, [&]() {
    dz_inplace_kernel(static_cast<uint16_t*>(slab), ld, static_cast<int>(rows), static_cast<int>(vocab), fmt, target,
                      vocab_offset, lse, c1, c2, c3, col_weight, inv_softcap, active_rows, active_base);
  });
  return 0;
}

// the ordered sums over all rows at the end of flce_b200_forward_backward
int emu_reduce_rows(long long n_rows, const float* loss_rows, const float* z_rows, const float* correct_rows, const float* norm,
                    float* scalars) {
  emu::launch(1, kRedThreads, [&]() {
    reduce_rows_kernel(static_cast<int>(n_rows), loss_rows, z_rows, correct_rows, norm, scalars);
  });
  return 0;
}

// bias gradient: column sums of a 16-bit slab, optionally accumulated
int emu_colsum(const void* dz, long long ld, long long rows, long long cols, int fmt, float* out, int accumulate,
               const int* active_rows, int active_base) {
  emu::launch(static_cast<unsigned>(ceil_div(cols, 64)), 1024, [&]() {
    colsum_accumulate_kernel(static_cast<const uint16_t*>(dz), ld, static_cast<int>(rows), static_cast<int>(cols), fmt, out,
                             accumulate, active_rows, active_base);
  });
  return 0;
}

// flce_b200_scale_gradient (grid of 148 * 8 blocks)
int emu_scale_inplace(void* data, long long n, int fmt, const float* scale) {
  emu::launch_serial(148 * 8, 256, [&]() { scale_inplace_kernel(data, n, fmt, scale); });
  return 0;
}

// per-(row, tile) partials -> row statistics (geometry of flce_b200_forward_stats)
int emu_merge_partials(long long n_rows, int n_tiles, const float* pmax, const float* psum, const float* plogit_sum,
                       const float* pamax_val, const int* pamax_idx, float* rowstats) {
  const int threads = 256;
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_rows, threads)), threads, [&]() {
    merge_partials_kernel(static_cast<int>(n_rows), n_tiles, pmax, psum, plogit_sum, pamax_val, pamax_idx, rowstats);
  });
  return 0;
}

// flce_b200_scaled_ce_rows / _grad / flce_b200_jsd_rows
int emu_scaled_ce_rows(const void* logits, long long ld, int dtype, long long n_rows, long long vocab, const long long* target,
                       long long ignore_index, float temperature, float* nll, float* entropy, float* lse) {
  const float inv_t = 1.f / temperature;
  if (dtype == 2) run_scaled_ce_rows<float>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, nll, entropy, lse);
  else if (dtype == 0) run_scaled_ce_rows<__nv_bfloat16>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, nll, entropy, lse);
  else run_scaled_ce_rows<__half>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, nll, entropy, lse);
  return 0;
}

int emu_scaled_ce_grad(void* logits, long long ld, int dtype, long long n_rows, long long vocab, const long long* target,
                       long long ignore_index, float temperature, const float* lse, const float* entropy, const float* g_nll,
                       const float* g_ent) {
  const float inv_t = 1.f / temperature;
  if (dtype == 2) run_scaled_ce_grad<float>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, lse, entropy, g_nll, g_ent);
  else if (dtype == 0) run_scaled_ce_grad<__nv_bfloat16>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, lse, entropy, g_nll, g_ent);
  else run_scaled_ce_grad<__half>(logits, ld, dtype, n_rows, vocab, target, ignore_index, inv_t, lse, entropy, g_nll, g_ent);
  return 0;
}

int emu_jsd_rows(void* student, long long ld_s, const void* teacher, long long ld_t, int dtype, long long n_rows, long long vocab,
                 const long long* labels, long long ignore_index, float beta, float temperature, const float* count,
                 float fixed_count, float* loss_rows) {
  const float inv_t = 1.f / temperature;
  if (dtype == 2) run_jsd_rows<float>(student, ld_s, teacher, ld_t, dtype, n_rows, vocab, labels, ignore_index, beta, inv_t, count, fixed_count, loss_rows);
  else if (dtype == 0) run_jsd_rows<__nv_bfloat16>(student, ld_s, teacher, ld_t, dtype, n_rows, vocab, labels, ignore_index, beta, inv_t, count, fixed_count, loss_rows);
  else run_jsd_rows<__half>(student, ld_s, teacher, ld_t, dtype, n_rows, vocab, labels, ignore_index, beta, inv_t, count, fixed_count, loss_rows);
  return 0;
}

// The persistent kernel's walk over the tile space: unit u visits tiles u, u + num_units, ... (gemm_sm100.cuh); visits[mt *
// n_tiles + nt] counts how often a tile is reached, order[] lists the tile ids in the order unit 0 sees them.
int emu_tile_schedule(int m_tiles, int n_tiles, int group, int group_along_m, int num_units, int* visits, int* order_unit0) {
  GemmShape shape{};
  shape.m_tiles = m_tiles;
  shape.n_tiles = n_tiles;
  shape.group = group;
  shape.group_along_m = group_along_m;
  const int num_tiles = m_tiles * n_tiles;
  int n0 = 0;
  for (int unit = 0; unit < num_units; ++unit)
    for (int tile = unit; tile < num_tiles; tile += num_units) {
      int mt = -1, nt = -1;
      decode_tile(shape, tile, mt, nt);
      if (mt < 0 || mt >= m_tiles || nt < 0 || nt >= n_tiles) return 1;
      ++visits[mt * n_tiles + nt];
      if (unit == 0) order_unit0[n0++] = mt * n_tiles + nt;
    }
  return 0;
}

// limit_to_active_rows: out[0] = m_tiles, out[1] = k_blocks after the adjustment
int emu_limit_to_active_rows(int m_tiles, int k_blocks, int role, int active_rows, int ctas_per_tile, int* out) {
  GemmShape shape{};
  shape.m_tiles = m_tiles;
  shape.k_blocks = k_blocks;
  shape.active_role = role;
  limit_to_active_rows(shape, active_rows, ctas_per_tile);
  out[0] = shape.m_tiles;
  out[1] = shape.k_blocks;
  return 0;
}

// sweep 1 (StatsEpilogue): per-(tile, row) partials, target logit, optional 16-bit copy of the soft-capped logits.
// Plane pointers may be null as in the library; target_logit must be zeroed by the caller (the library memsets it).
int emu_sweep_stats(const void* x, const void* w, int dtype, int m, int vocab, int k, long long ld_x, long long ld_w,
                    const long long* target, const float* bias, const float* col_weight, float softcap, long long vocab_offset,
                    float* pmax, float* psum, float* plogit_sum, float* pamax_val, int* pamax_idx, float* target_logit,
                    void* logits_out, long long ld_logits, int logits_fmt, int m_tile_limit, const float* shift,
                    long long ignore_index) {
  StatsEpilogue::Params ep{};
  ep.target = target;
  ep.bias = bias;
  ep.col_weight = col_weight;
  ep.softcap = softcap;
  ep.inv_softcap = softcap > 0.f ? 1.f / softcap : 0.f;
  ep.n_cols = vocab;
  ep.vocab_offset = vocab_offset;
  ep.m_rows = m;
  ep.pmax = pmax;
  ep.psum = psum;
  ep.plogit_sum = plogit_sum;
  ep.pamax_val = pamax_val;
  ep.pamax_idx = pamax_idx;
  ep.target_logit = target_logit;
  ep.logits_out = logits_out;
  ep.ld_logits = ld_logits;
  ep.logits_fmt = logits_fmt;
  ep.shift = shift;
  ep.ignore_index = ignore_index;
  run_tiles<StatsEpilogue>(ep, x, w, dtype, m, vocab, k, ld_x, ld_w, m_tile_limit);
  return 0;
}

// sweep 2 (DzEpilogue): the 16-bit logit-gradient slab (and the optional rounding-residual slab)
int emu_sweep_dz(const void* x, const void* w, int dtype, int m, int vocab, int k, long long ld_x, long long ld_w,
                 const long long* target, const float* bias, const float* col_weight, float softcap, long long vocab_offset,
                 const float* lse, const float* c1, const float* c2, const float* c3, void* dz, void* dz_lo, long long ld_dz,
                 int out_fmt, int m_tile_limit) {
  DzEpilogue::Params ep;
  ep.target = target;
  ep.bias = bias;
  ep.col_weight = col_weight;
  ep.softcap = softcap;
  ep.inv_softcap = softcap > 0.f ? 1.f / softcap : 0.f;
  ep.n_cols = vocab;
  ep.vocab_offset = vocab_offset;
  ep.m_rows = m;
  ep.lse = lse;
  ep.c1 = c1;
  ep.c2 = c2;
  ep.c3 = c3;
  ep.dz = dz;
  ep.dz_lo = dz_lo;
  ep.ld_dz = ld_dz;
  ep.out_fmt = out_fmt;
  run_tiles<DzEpilogue>(ep, x, w, dtype, m, vocab, k, ld_x, ld_w, m_tile_limit);
  return 0;
}

// StoreEpilogue: D = A . B^T (+ acc) with both operands K-major; acc (fp32, in/out) and out (out_fmt) may each be null
int emu_gemm_store(const void* a, const void* b, int dtype, int m, int n, int k, long long ld_a, long long ld_b, float* acc,
                   long long ld_acc, void* out, long long ld_out, int out_fmt) {
  StoreEpilogue::Params ep{};
  ep.m_rows = m;
  ep.n_cols = n;
  ep.acc_in = acc;
  ep.acc_out = acc;
  ep.ld_acc = ld_acc;
  ep.out = out;
  ep.ld_out = ld_out;
  ep.out_fmt = out_fmt;
  run_tiles_store(ep, a, b, dtype, m, n, k, ld_a, ld_b, kBlockN);
  return 0;
}

// StoreEpilogue with every option: separate fp32 partial in / out, per-row scale, rank-1 correction (all nullable)
int emu_gemm_store_ex(const void* a, const void* b, int dtype, int m, int n, int k, long long ld_a, long long ld_b,
                      const float* acc_in, float* acc_out, long long ld_acc, void* out, long long ld_out, int out_fmt,
                      const float* row_scale, const float* r1_row, const float* r1_col, int acc_add) {
  StoreEpilogue::Params ep{};
  ep.m_rows = m;
  ep.n_cols = n;
  ep.acc_in = acc_in;
  ep.acc_out = acc_out;
  ep.ld_acc = ld_acc;
  ep.out = out;
  ep.ld_out = ld_out;
  ep.out_fmt = out_fmt;
  ep.row_scale = row_scale;
  ep.r1_row = r1_row;
  ep.r1_col = r1_col;
  ep.acc_add = acc_add;
  ep.bulk = (acc_in == nullptr && ((out != nullptr) != (acc_out != nullptr))) ? 1 : 0;   // the launcher's rule
  run_tiles_store(ep, a, b, dtype, m, n, k, ld_a, ld_b, 2 * kBlockN);   // the 512-column tile of the gradient GEMMs
  return 0;
}

// fp32 accumulator -> 16-bit weight gradient after the last token chunk
int emu_convert_f32(const float* src, long long n, int fmt, void* dst) {
  emu::launch_serial(8, 256, [&]() { convert_f32_kernel(src, n, fmt, static_cast<uint16_t*>(dst)); });
  return 0;
}

// the exp-store form of the single-sweep mode: reference points, per-chunk fix-up, ordered scaled column sums
// (launch geometry of flce_b200_forward_backward)
int emu_target_shift(const void* x, long long ld_x, const void* w, long long ld_w, int fmt, int n_rows, int hidden,
                     const long long* target, long long ignore_index, long long vocab, long long vocab_offset, int sharded,
                     const float* bias, float softcap, float* shift) {
  const int warps = 8;
  emu::launch(static_cast<unsigned>(ceil_div(n_rows, warps)), warps * 32, [&]() {
    target_shift_kernel(static_cast<const uint16_t*>(x), ld_x, static_cast<const uint16_t*>(w), ld_w, fmt, n_rows, hidden,
                        target, ignore_index, vocab, vocab_offset, sharded, bias, softcap, softcap > 0.f ? 1.f / softcap : 0.f,
                        kExpStoreOffset, shift);
  });
  return 0;
}

int emu_shift_fill(int n_rows, float* shift) {
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_rows, 256)), 256, [&]() { shift_fill_kernel(n_rows, kExpStoreOffset, shift); });
  return 0;
}

int emu_exp_store_fixup(const void* x, long long ld_x, int hidden, int fmt, int n_rows, const long long* target,
                        long long ignore_index, long long vocab, long long vocab_offset, const float* lse, const float* shift,
                        const float* target_logit, const float* c1, const float* c3, float softcap, void* slab,
                        long long ld_slab, float* alpha, void* xs, long long ld_xs) {
  emu::launch_serial(static_cast<unsigned>(n_rows), 256, [&]() {
    exp_store_fixup_kernel(static_cast<const uint16_t*>(x), ld_x, hidden, fmt, n_rows, target, ignore_index, vocab, vocab_offset, lse, shift,
                           target_logit, c1, c3, softcap > 0.f ? 1.f / softcap : 0.f, kExpStoreClamp,
                           static_cast<uint16_t*>(slab), ld_slab, alpha, static_cast<uint16_t*>(xs), ld_xs);
  });
  return 0;
}

// returns the chunk's redo flag; when it is raised the reference points have been moved onto the log-sum-exp
int emu_exp_store_check(int n_rows, const long long* target, long long ignore_index, const float* lse, float* shift) {
  int flag = 0;
  const int threads = 256;
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_rows, threads)), threads, [&]() {
    exp_store_check_kernel(n_rows, target, ignore_index, lse, shift, kExpStoreRedoLimit, &flag);
  });
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_rows, threads)), threads, [&]() {
    exp_store_reshift_kernel(n_rows, lse, &flag, shift);
  });
  return flag;
}

int emu_scaled_colsum(const void* mat, long long ld, int n_rows, int n_cols, int fmt, const float* scale, float* scratch,
                      float* out, int accumulate) {
  const emu::Dim3 grid(static_cast<unsigned>(ceil_div(n_cols, 64)), kColsumSplits, 1);
  emu::launch(grid, 1024, [&]() {
    scaled_colsum_stage1_kernel(static_cast<const uint16_t*>(mat), ld, n_rows, n_cols, fmt, scale, scratch);
  });
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_cols, 256)), 256, [&]() {
    scaled_colsum_stage2_kernel(scratch, n_cols, out, accumulate);
  });
  return 0;
}

// coefficients of the logit gradient (coef_kernel, geometry of flce_b200_backward)
int emu_coef(long long n_rows, long long ignore_index, float alpha, float lambda, int mean, int token_scaling, long long vocab,
             long long vocab_total, long long vocab_offset, const long long* target, const float* ce_weight, const float* lse,
             const float* prob, const float* norm, const float* grad_output, int per_row, float* c1, float* c2, float* c3) {
  RowMath rm;
  rm.ignore_index = ignore_index;
  rm.alpha = alpha;
  rm.eps = alpha / static_cast<float>(vocab_total);
  rm.lambda = lambda;
  rm.mean = mean;
  rm.token_scaling = token_scaling;
  rm.weighted = ce_weight != nullptr;
  rm.vocab = vocab;
  rm.vocab_offset = vocab_offset;
  const int threads = 256;
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_rows, threads)), threads, [&]() {
    coef_kernel(static_cast<int>(n_rows), rm, target, ce_weight, lse, prob, norm, grad_output, per_row, c1, c2, c3);
  });
  return 0;
}

// per-row loss and metrics (finalize_rows_kernel + reduce_rows_kernel, geometry of flce_b200_forward_finalize)
int emu_finalize(long long n_rows, long long ignore_index, float alpha, float lambda, int mean, int token_scaling, long long vocab,
                 long long vocab_total, long long vocab_offset, const long long* target, const float* ce_weight,
                 const float* rowstats, const float* norm, float* lse, float* prob, float* loss_rows, float* z_rows,
                 float* correct_rows, long long* predicted, float* scalars) {
  RowMath rm;
  rm.ignore_index = ignore_index;
  rm.alpha = alpha;
  rm.eps = alpha / static_cast<float>(vocab_total);
  rm.lambda = lambda;
  rm.mean = mean;
  rm.token_scaling = token_scaling;
  rm.weighted = ce_weight != nullptr;
  rm.vocab = vocab;
  rm.vocab_offset = vocab_offset;
  const int threads = 256;
  emu::launch_serial(static_cast<unsigned>(ceil_div(n_rows, threads)), threads, [&]() {
    finalize_rows_kernel(static_cast<int>(n_rows), rm, target, ce_weight, rowstats, norm, lse, prob, loss_rows, z_rows,
                         correct_rows, predicted);
  });
  if (scalars != nullptr)
    emu::launch(1, kRedThreads, [&]() {
      reduce_rows_kernel(static_cast<int>(n_rows), loss_rows, z_rows, correct_rows, norm, scalars);
    });
  return 0;
}

// scaled cross-entropy on the two sweeps: EntropyStatsEpilogue + scaled_ce_merge_kernel (flce_b200_sce_forward) ...
int emu_sce_forward(const void* x, const void* w, int dtype, int m, int vocab, int k, long long ld_x, long long ld_w,
                    const long long* target, long long ignore_index, float temperature, float* planes, float* target_logit,
                    float* nll, float* entropy, float* lse) {
  const int n_tiles = static_cast<int>(ceil_div(vocab, kBlockN));
  const size_t plane = static_cast<size_t>(n_tiles) * m;
  EntropyStatsEpilogue::Params ep{};
  ep.target = target;
  ep.scale = 1.f / temperature;
  ep.n_cols = vocab;
  ep.m_rows = m;
  ep.pmax = planes;
  ep.psum = planes + plane;
  ep.pts = planes + 2 * plane;
  ep.target_logit = target_logit;
  run_tiles<EntropyStatsEpilogue>(ep, x, w, dtype, m, vocab, k, ld_x, ld_w);
  const int threads = 256;
  emu::launch_serial(static_cast<unsigned>(ceil_div(m, threads)), threads, [&]() {
    scaled_ce_merge_kernel(m, n_tiles, ep.pmax, ep.psum, ep.pts, target_logit, target, ignore_index, nll, entropy, lse);
  });
  return 0;
}

// ... and ScaledDzEpilogue over one vocabulary slab (the logit-gradient step of flce_b200_sce_backward); w points at the
// slab's first row, vocab_offset is that row's class id
int emu_sce_sweep_dz(const void* x, const void* w, int dtype, int m, int cols, int k, long long ld_x, long long ld_w,
                     const long long* target, long long ignore_index, float temperature, long long vocab_offset, const float* lse,
                     const float* entropy, const float* g_nll, const float* g_ent, void* dz, long long ld_dz, int out_fmt) {
  ScaledDzEpilogue::Params ep;
  ep.target = target;
  ep.ignore_index = ignore_index;
  ep.scale = 1.f / temperature;
  ep.n_cols = cols;
  ep.vocab_offset = vocab_offset;
  ep.m_rows = m;
  ep.lse = lse;
  ep.entropy = entropy;
  ep.grad_nll = g_nll;
  ep.grad_entropy = g_ent;
  ep.dz = dz;
  ep.ld_dz = ld_dz;
  ep.out_fmt = out_fmt;
  run_tiles<ScaledDzEpilogue>(ep, x, w, dtype, m, cols, k, ld_x, ld_w);
  return 0;
}

}  // extern "C"
