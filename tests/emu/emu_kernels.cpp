// The library's SIMT kernels (csrc/row_kernels.cuh, csrc/ce_kernels.cuh, csrc/head_loss_kernels.cuh) compiled for the host and run on the host
// through simt_emulation.hpp, behind a small C interface for the CPU tests.  Every wrapper repeats the launch geometry
// and kernel order of the library entry point it is named after (csrc/flce_b200.cu), so the tests exercise the same
// index arithmetic a GPU launch would.  ex2.approx / rcp.approx are replaced by libm (FLCE_HOST_EMULATION), so results
// agree with the GPU to a few ulp, not bit for bit.
//
// Test infrastructure only.
#define FLCE_HOST_EMULATION 1
#include "simt_emulation.hpp"

#include "ce_kernels.cuh"
#include "head_loss_kernels.cuh"
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
                       static_cast<unsigned>(ceil_div(ceil_div(p.vocab, per_thread), kCeThreads)), 1);
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
  emu::launch(emu::Dim3(static_cast<unsigned>(n_rows)), emu::Dim3(kCeThreads), [&]() {
    if (vec)
      jsd_rows_kernel<T, true>(xs, ld_s, xt, ld_t, static_cast<int>(n_rows), static_cast<int>(vocab), labels, ignore_index, beta,
                               inv_t, count, fixed_count, loss_rows);
    else
      jsd_rows_kernel<T, false>(xs, ld_s, xt, ld_t, static_cast<int>(n_rows), static_cast<int>(vocab), labels, ignore_index, beta,
                                inv_t, count, fixed_count, loss_rows);
  });
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
                   const float* col_weight, float inv_softcap) {
  const int tpb = 256;
  const emu::Dim3 grid(static_cast<unsigned>(ceil_div(ceil_div(vocab, 8), tpb)), static_cast<unsigned>(rows), 1);
  emu::launch_serial(grid, tpb, [&]() {
    dz_inplace_kernel(static_cast<uint16_t*>(slab), ld, static_cast<int>(rows), static_cast<int>(vocab), fmt, target,
                      vocab_offset, lse, c1, c2, c3, col_weight, inv_softcap);
  });
  return 0;
}

// bias gradient: column sums of a 16-bit slab, optionally accumulated
int emu_colsum(const void* dz, long long ld, long long rows, long long cols, int fmt, float* out, int accumulate) {
  emu::launch(static_cast<unsigned>(ceil_div(cols, 64)), 1024, [&]() {
    colsum_accumulate_kernel(static_cast<const uint16_t*>(dz), ld, static_cast<int>(rows), static_cast<int>(cols), fmt, out,
                             accumulate);
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

}  // extern "C"
