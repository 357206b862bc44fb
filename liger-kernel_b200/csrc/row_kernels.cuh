// The SIMT kernels around the tensor-core sweeps: target counting, merging of per-tile softmax partials, per-row loss
// and gradient coefficients, ordered reductions, the in-place logit gradient of the single-sweep mode, column sums,
// row compaction for ignored tokens and the fp32 -> 16-bit term split.  All HBM- or latency-bound; none touches
// tensor memory, so this header also compiles for the host emulation the CPU tests use.
#pragma once

#include "simt_common.cuh"

namespace flce {

constexpr int kRedThreads = 1024;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  // fixed-order tree: deterministic for a given block size
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = 0.f;
  if (warp == 0) {
    r = (lane < (blockDim.x >> 5)) ? scratch[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  return r;  // valid in warp 0
}

// norm[0] = #rows with target != ignore_index, norm[1] = sum of class weight of those targets,
// norm[2] = sum of all class weights (vocab_total when unweighted), norm[3] = #targets outside [0, vocab_total).
// One block: exact and ordered.
__global__ void count_kernel(const long long* target, long long n_rows, long long ignore_index, const float* ce_weight,
                             long long vocab, long long vocab_offset, float vocab_total, float* norm) {
  __shared__ float scratch[32];
  float cnt = 0.f, wy = 0.f, wall = 0.f, bad = 0.f;
  const long long classes = static_cast<long long>(vocab_total);
  for (long long i = threadIdx.x; i < n_rows; i += blockDim.x) {
    const long long t = target[i];
    if (t != ignore_index) {
      cnt += 1.f;
      if (t < 0 || t >= classes) bad += 1.f;   // matches no class; reported, never dereferenced
      if (ce_weight != nullptr) {
        const long long l = t - vocab_offset;
        if (l >= 0 && l < vocab) wy += ce_weight[l];
      }
    }
  }
  if (ce_weight != nullptr)
    for (long long j = threadIdx.x; j < vocab; j += blockDim.x) wall += ce_weight[j];
  const float c = block_sum(cnt, scratch);
  const float w = block_sum(wy, scratch);
  const float a = block_sum(wall, scratch);
  const float o = block_sum(bad, scratch);
  if (threadIdx.x == 0) {
    norm[0] = c;
    norm[1] = (ce_weight != nullptr) ? w : c;
    norm[2] = (ce_weight != nullptr) ? a : vocab_total;
    norm[3] = o;
  }
}

// per-(row, tile) partials -> per-row statistics planes
__global__ void merge_partials_kernel(int m_rows, int n_tiles, const float* pmax, const float* psum,
                                      const float* plogit_sum, const float* pamax_val, const int* pamax_idx,
                                      float* rowstats) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= m_rows) return;
  float m = -INFINITY;
  for (int t = 0; t < n_tiles; ++t) m = fmaxf(m, pmax[static_cast<size_t>(t) * m_rows + row]);
  float d = 0.f, ss = 0.f, best = -INFINITY;
  int best_idx = 0;
  for (int t = 0; t < n_tiles; ++t) {
    const size_t o = static_cast<size_t>(t) * m_rows + row;
    d += psum[o] * expf(pmax[o] - m);
    if (plogit_sum != nullptr) ss += plogit_sum[o];
    if (pamax_val != nullptr) {
      const float v = pamax_val[o];
      if (v > best) {
        best = v;
        best_idx = pamax_idx[o];
      }
    }
  }
  const size_t n = static_cast<size_t>(m_rows);
  rowstats[0 * n + row] = m;
  rowstats[1 * n + row] = d;
  // plane 2 (target logit) was written by the sweep itself
  rowstats[3 * n + row] = ss;
  rowstats[4 * n + row] = best;
  reinterpret_cast<int*>(rowstats)[5 * n + row] = best_idx;
}

struct RowMath {
  long long ignore_index;
  float alpha, eps, lambda;
  int mean, token_scaling, weighted;
  long long vocab, vocab_offset;
};

// per-row loss / metrics (src/liger_kernel/ops/cross_entropy.py:289-336 of the reference) from the row's statistics:
// m, d = running maximum and sum of exponentials, xy = target logit, ss = (weighted) logit sum, amax = arg-max
__device__ __forceinline__ void finalize_row(int row, const RowMath& rm, long long t, const float* ce_weight, float m, float d,
                                             float xy, float ss, int amax, const float* norm, float* lse_out, float* prob_out,
                                             float* loss_rows, float* z_rows, float* correct_rows, long long* predicted) {
  const bool valid = t != rm.ignore_index;
  const float lse = m + logf(d);
  if (lse_out != nullptr) lse_out[row] = lse;
  float loss = 0.f, z = 0.f, py = 0.f, correct = 0.f;
  long long pred = -1;
  if (valid) {
    float wy = 1.f;
    if (rm.weighted) {
      const long long l = t - rm.vocab_offset;
      wy = (l >= 0 && l < rm.vocab) ? ce_weight[l] : 0.f;
    }
    loss = (lse - xy) * wy;
    if (rm.alpha > 0.f) {
      const float smooth = -rm.eps * ss + (rm.weighted ? rm.eps * lse * norm[2] : rm.alpha * lse);
      loss = loss * (1.f - rm.alpha) + smooth;
    }
    z = rm.lambda * lse * lse;
    if (rm.mean) {
      loss /= norm[1];
      z /= norm[0];
    }
    loss += z;
    py = expf(xy - lse);
    if (rm.token_scaling) {
      loss *= py;
      z *= py;
    }
    pred = amax;
    correct = (static_cast<long long>(amax) == t) ? 1.f : 0.f;
  }
  if (prob_out != nullptr) prob_out[row] = py;
  if (loss_rows != nullptr) loss_rows[row] = loss;
  if (z_rows != nullptr) z_rows[row] = z;
  if (correct_rows != nullptr) correct_rows[row] = correct;
  if (predicted != nullptr) predicted[row] = pred;
}

__global__ void finalize_rows_kernel(int m_rows, RowMath rm, const long long* target, const float* ce_weight,
                                     const float* rowstats, const float* norm, float* lse_out, float* prob_out,
                                     float* loss_rows, float* z_rows, float* correct_rows, long long* predicted) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= m_rows) return;
  const size_t n = static_cast<size_t>(m_rows);
  finalize_row(row, rm, target[row], ce_weight, rowstats[0 * n + row], rowstats[1 * n + row], rowstats[2 * n + row],
               rowstats[3 * n + row], reinterpret_cast<const int*>(rowstats)[5 * n + row], norm, lse_out, prob_out, loss_rows,
               z_rows, correct_rows, predicted);
}

// scalars[0] = sum loss_rows, [1] = sum z_rows, [2] = sum correct / n_non_ignore, [3] = n_non_ignore
__global__ void reduce_rows_kernel(int m_rows, const float* loss_rows, const float* z_rows, const float* correct_rows,
                                   const float* norm, float* scalars) {
  __shared__ float scratch[32];
  float a = 0.f, b = 0.f, c = 0.f;
  for (int i = threadIdx.x; i < m_rows; i += blockDim.x) {
    if (loss_rows != nullptr) a += loss_rows[i];
    if (z_rows != nullptr) b += z_rows[i];
    if (correct_rows != nullptr) c += correct_rows[i];
  }
  const float sa = block_sum(a, scratch);
  const float sb = block_sum(b, scratch);
  const float sc = block_sum(c, scratch);
  if (threadIdx.x == 0) {
    scalars[0] = sa;
    scalars[1] = sb;
    scalars[2] = sc / norm[0];
    scalars[3] = norm[0];
  }
}

// per-row coefficients of the logit gradient (see DzEpilogue): go = upstream gradient of the row, prob = exp(xy - lse)
__device__ __forceinline__ void row_coefs(const RowMath& rm, long long t, const float* ce_weight, float lse, float prob,
                                          const float* norm, float go, float& a, float& b, float& c) {
  a = b = c = 0.f;
  if (t == rm.ignore_index) return;
  if (rm.token_scaling) go *= prob;
  float wy = 1.f;
  if (rm.weighted) {
    const long long l = t - rm.vocab_offset;
    wy = (l >= 0 && l < rm.vocab) ? ce_weight[l] : 0.f;
  }
  const float inv_s = rm.mean ? 1.f / norm[1] : 1.f;
  const float inv_n = rm.mean ? 1.f / norm[0] : 1.f;
  const float sum_w = norm[2];
  a = go * (((1.f - rm.alpha) * wy + rm.eps * sum_w) * inv_s + 2.f * rm.lambda * lse * inv_n);
  b = go * rm.eps * inv_s;
  c = go * (1.f - rm.alpha) * wy * inv_s;
}

__global__ void coef_kernel(int m_rows, RowMath rm, const long long* target, const float* ce_weight, const float* lse,
                            const float* prob, const float* norm, const float* grad_output, int per_row, float* c1,
                            float* c2, float* c3) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= m_rows) return;
  float go = 1.f;
  if (grad_output != nullptr) go = per_row ? grad_output[row] : grad_output[0];
  float a, b, c;
  row_coefs(rm, target[row], ce_weight, lse[row], rm.token_scaling ? prob[row] : 0.f, norm, go, a, b, c);
  c1[row] = a;
  c2[row] = b;
  c3[row] = c;
}

// Single-sweep mode: turn the stored 16-bit soft-capped logits of a token chunk into the logit gradient, in place.
//   dZ = (exp(s - lse) * c1 - c2 * colw - c3 * [j == target]) * (1 - (s/softcap)^2)
// One block per (row, segment of kDzInplaceCols columns); every thread issues its four 16-byte loads before it touches
// any of them, so that enough bytes are in flight to fill HBM (reads and writes each element once).  With active_rows
// given, only the first *active_rows - active_base rows matter; the weight-gradient GEMM still reads whole 64-row K
// slices, so the rows up to the next multiple of 64 are turned into gradients too (zeros: their coefficients are
// zero and the sweep wrote their logits), and the rest, which nothing reads, is skipped.
constexpr int kDzInplaceThreads = 256;
constexpr int kDzInplaceVecs = 4;
constexpr int kDzInplaceCols = kDzInplaceThreads * kDzInplaceVecs * 8;
__global__ void __launch_bounds__(kDzInplaceThreads)
dz_inplace_kernel(uint16_t* slab, long long ld, int n_rows, int n_cols, int fmt, const long long* target,
                  long long vocab_offset, const float* lse, const float* c1, const float* c2, const float* c3,
                  const float* col_weight, float inv_softcap, const int* active_rows = nullptr, int active_base = 0) {
  const int row = blockIdx.y;
  if (row >= n_rows) return;
  if (active_rows != nullptr && row >= (max(0, *active_rows - active_base) + 63) / 64 * 64) return;
  const float l2 = lse[row] * kLog2e, a = c1[row], b = c2[row], c = c3[row];
  const long long t = target[row] - vocab_offset;
  uint16_t* row_ptr = slab + static_cast<size_t>(row) * ld;
  const int col0 = blockIdx.x * kDzInplaceCols + threadIdx.x * 8;
  uint4 raw[kDzInplaceVecs];
#pragma unroll
  for (int v = 0; v < kDzInplaceVecs; ++v) {
    const int col = col0 + v * kDzInplaceThreads * 8;
    if (col < n_cols) raw[v] = *reinterpret_cast<const uint4*>(row_ptr + col);
  }
#pragma unroll
  for (int v = 0; v < kDzInplaceVecs; ++v) {
    const int col = col0 + v * kDzInplaceThreads * 8;
    if (col >= n_cols) continue;
    const uint32_t words[4] = {raw[v].x, raw[v].y, raw[v].z, raw[v].w};
    float g[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 f;
      if (fmt == kOutBf16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[q]));
      else f = __half22float2(*reinterpret_cast<const __half2*>(&words[q]));
      g[2 * q] = f.x;
      g[2 * q + 1] = f.y;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = g[j];
      const float wj = (col_weight != nullptr && col + j < n_cols) ? col_weight[col + j] : 1.f;
      float val = fmaf(ex2_approx(fmaf(s, kLog2e, -l2)), a, -b * wj);
      if (static_cast<long long>(col + j) == t) val -= c;
      if (inv_softcap > 0.f) {
        const float th = s * inv_softcap;
        val *= fmaf(-th, th, 1.f);
      }
      g[j] = (col + j < n_cols) ? val : 0.f;
    }
    uint4 o;
    o.x = pack2(g[0], g[1], fmt);
    o.y = pack2(g[2], g[3], fmt);
    o.z = pack2(g[4], g[5], fmt);
    o.w = pack2(g[6], g[7], fmt);
    *reinterpret_cast<uint4*>(row_ptr + col) = o;
  }
}

// ---- the exp-store form of the single-sweep mode ----------------------------------------------------------------
// Sweep 1 stores E = exp(s - shift) (epilogues.cuh) instead of the logits.  The three kernels below produce the per-row
// reference point before the sweep, and, once the chunk's log-sum-exp is known, everything the two gradient GEMMs
// need so that they can consume E as it is:  dZ[r, j] = alpha_r * E[r, j]  with  alpha_r = c1_r * exp(shift_r - lse_r).

__device__ __forceinline__ float dot8_16bit(const uint4& a, const uint4& b, int fmt) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  float acc = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float2 fa, fb;
    if (fmt == kOutBf16) {
      fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[q]));
      fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[q]));
    } else {
      fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[q]));
      fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[q]));
    }
    acc = fmaf(fa.x, fb.x, acc);
    acc = fmaf(fa.y, fb.y, acc);
  }
  return acc;
}

// shift[r] = soft-capped logit of row r's target class + offset: x_r . W[y_r] (+ bias), one warp per row.
// The log-sum-exp of a row is at least its target logit and exceeds it by the row's loss, so this point is within
// [offset - loss, offset] of it without a pass over the vocabulary.  Rows without a usable target get the offset alone.
// On a vocabulary shard (sharded != 0; w holds classes [vocab_offset, vocab_offset + vocab)) rows whose target lives
// elsewhere get -inf: the caller takes the maximum over the shards and shift_fill_kernel settles the rows no shard owns.
__global__ void target_shift_kernel(const uint16_t* x, long long ld_x, const uint16_t* w, long long ld_w, int fmt, int n_rows,
                                    int hidden, const long long* target, long long ignore_index, long long vocab,
                                    long long vocab_offset, int sharded, const float* bias, float softcap, float inv_softcap,
                                    float offset, float* shift) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const long long t = target[row];
  const long long y = t - vocab_offset;
  float z = 0.f;
  if (t != ignore_index && y >= 0 && y < vocab) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ld_x);
    const uint4* wr = reinterpret_cast<const uint4*>(w + static_cast<size_t>(y) * ld_w);
    float acc = 0.f;
    for (int v = lane; v < hidden / 8; v += 32) acc += dot8_16bit(xr[v], wr[v], fmt);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    z = acc + (bias != nullptr ? bias[y] : 0.f);
    if (softcap > 0.f) z = softcap * tanh_accurate(z * inv_softcap);
  } else if (sharded) {
    z = -INFINITY;
  }
  if (lane == 0) shift[row] = z + offset;
}
// rows whose target no shard owns (ignore_index, out of range): the offset alone, as in the unsharded case
__global__ void shift_fill_kernel(int n_rows, float offset, float* shift) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < n_rows && !(shift[row] > -3.0e38f)) shift[row] = offset;
}

// The stored exponentials are exact only while exp(s - shift) stays inside the clamp and the per-row factor inside fp32:
// a row whose log-sum-exp lies more than `limit` above shift - offset (a loss of that many nats) breaks that.  The
// first kernel raises *flag when the chunk holds such a row, the second then moves every reference point of the chunk
// onto the now known log-sum-exp; sweep 1 is enqueued once more for the chunk, gated on the same flag.
__global__ void exp_store_check_kernel(int n_rows, const long long* target, long long ignore_index, const float* lse,
                                       const float* shift, float limit, int* flag) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n_rows || target[row] == ignore_index) return;
  if (!(lse[row] - shift[row] <= limit)) *flag = 1;   // also true for NaN: take the exact path
}
__global__ void exp_store_reshift_kernel(int n_rows, const float* lse, const int* flag, float* shift) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n_rows || *flag == 0) return;
  shift[row] = lse[row];
}

// One block per row of the chunk, after the chunk's coefficients are known:
//   alpha[r] = c1_r * exp(shift_r - lse_r)                          (0 on rows whose target is ignore_index)
//   xs[r, :] = 16-bit(alpha_r * x[r, :])                            (the weight-gradient GEMM's second operand)
//   E[r, y_r] = (exp(s_y - shift_r) - c3_r / alpha_r) * chain_y     (the true-class term, formed in fp32 from the fp32
//                                                                    target logit, not from the rounded stored value)
__global__ void exp_store_fixup_kernel(const uint16_t* x, long long ld_x, int hidden, int fmt, int n_rows,
                                       const long long* target, long long ignore_index, long long vocab,
                                       long long vocab_offset, const float* lse, const float* shift,
                                       const float* target_logit, const float* c1, const float* c3, float inv_softcap,
                                       float clamp, uint16_t* slab, long long ld_slab, float* alpha, uint16_t* xs,
                                       long long ld_xs) {
  const int row = blockIdx.x;
  if (row >= n_rows) return;
  const long long t = target[row];
  const long long y = t - vocab_offset;          // column of the target in this (shard of the) vocabulary, if it is here
  const bool live = t != ignore_index;
  const float a = live ? c1[row] * ex2_approx((shift[row] - lse[row]) * kLog2e) : 0.f;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ld_x);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(row) * ld_xs);
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) {
    const uint4 raw = src[v];
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 f;
      if (fmt == kOutBf16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[q]));
      else f = __half22float2(*reinterpret_cast<const __half2*>(&words[q]));
      o[q] = pack2(f.x * a, f.y * a, fmt);
    }
    dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (threadIdx.x == 0) {
    alpha[row] = a;
    if (live && y >= 0 && y < vocab) {
      const float sy = target_logit[row];
      float chain = 1.f;
      if (inv_softcap > 0.f) {
        const float th = sy * inv_softcap;
        chain = fmaf(-th, th, 1.f);
      }
      const float e = ex2_approx(fminf((sy - shift[row]) * kLog2e, clamp * kLog2e));
      const float val = (a != 0.f) ? (e - c3[row] / a) * chain : 0.f;
      if (fmt == kOutBf16) {
        const __nv_bfloat16 h = __float2bfloat16_rn(val);
        slab[static_cast<size_t>(row) * ld_slab + y] = *reinterpret_cast<const uint16_t*>(&h);
      } else {
        const __half h = __float2half_rn(val);
        slab[static_cast<size_t>(row) * ld_slab + y] = *reinterpret_cast<const uint16_t*>(&h);
      }
    }
  }
}

// out[c] (+)= sum over rows of scale[r] * mat[r, c] for a 16-bit matrix (scale null = 1), in two ordered stages:
// stage 1 (grid = column blocks of 64 x kColsumSplits row ranges) leaves partial sums in scratch[split][c],
// stage 2 adds them up in a fixed order.  Used for sum_j w_j W[j, :] and sum_r c2_r x[r, :] (label smoothing).
constexpr int kColsumSplits = 32;
__global__ void scaled_colsum_stage1_kernel(const uint16_t* mat, long long ld, int n_rows, int n_cols, int fmt, const float* scale,
                                            float* scratch) {
  __shared__ float part[16][64];
  const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;   // 64 x 16
  const int col = blockIdx.x * 64 + cx;
  const int per = (n_rows + kColsumSplits - 1) / kColsumSplits;
  const int r_begin = blockIdx.y * per, r_end = min(n_rows, r_begin + per);
  float s = 0.f;
  if (col < n_cols) {
    for (int r = r_begin + ry; r < r_end; r += 16) {
      const uint16_t raw = mat[static_cast<size_t>(r) * ld + col];
      const float v = (fmt == kOutBf16) ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                                        : __half2float(*reinterpret_cast<const __half*>(&raw));
      s = fmaf(scale != nullptr ? scale[r] : 1.f, v, s);
    }
  }
  part[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && col < n_cols) {
    float t = 0.f;
    for (int i = 0; i < 16; ++i) t += part[i][cx];
    scratch[static_cast<size_t>(blockIdx.y) * n_cols + col] = t;
  }
}
__global__ void scaled_colsum_stage2_kernel(const float* scratch, int n_cols, float* out, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= n_cols) return;
  float t = accumulate ? out[col] : 0.f;
  for (int i = 0; i < kColsumSplits; ++i) t += scratch[static_cast<size_t>(i) * n_cols + col];
  out[col] = t;
}

// fp32 accumulator -> 16-bit result, once every token chunk has added its part (single-sweep weight gradient)
__global__ void convert_f32_kernel(const float* src, long long n, int fmt, uint16_t* dst) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    if (i + 8 <= n) {
      const float4 a = *reinterpret_cast<const float4*>(src + i);
      const float4 b = *reinterpret_cast<const float4*>(src + i + 4);
      uint4 o;
      o.x = pack2(a.x, a.y, fmt);
      o.y = pack2(a.z, a.w, fmt);
      o.z = pack2(b.x, b.y, fmt);
      o.w = pack2(b.z, b.w, fmt);
      *reinterpret_cast<uint4*>(dst + i) = o;
    } else {
      for (long long j = i; j < n; ++j) {
        const uint32_t two = pack2(src[j], 0.f, fmt);
        dst[j] = static_cast<uint16_t>(two & 0xffffu);
      }
    }
  }
}

// data[i] *= *scale unless *scale == 1 (checked on the device: no host synchronisation); 16-bit or fp32 elements
__global__ void scale_inplace_kernel(void* data, long long n, int fmt, const float* scale) {
  const float s = *scale;
  if (s == 1.f) return;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (fmt == kOutFp32) {
      static_cast<float*>(data)[i] *= s;
    } else if (fmt == kOutBf16) {
      __nv_bfloat16* p = static_cast<__nv_bfloat16*>(data) + i;
      *p = __float2bfloat16_rn(__bfloat162float(*p) * s);
    } else {
      __half* p = static_cast<__half*>(data) + i;
      *p = __float2half_rn(__half2float(*p) * s);
    }
  }
}

// out[j] += sum over rows of slab column j (bias gradient across token chunks); one block per 64 columns
// (rows at and beyond *active_rows, when given, were never written by the sweep and are left out)
__global__ void colsum_accumulate_kernel(const uint16_t* dz, long long ld, int m_rows, int n_cols, int fmt, float* out,
                                         int accumulate, const int* active_rows = nullptr, int active_base = 0) {
  __shared__ float part[16][64];
  if (active_rows != nullptr) m_rows = min(m_rows, max(0, *active_rows - active_base));
  const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;
  const int col = blockIdx.x * 64 + cx;
  float s = 0.f;
  if (col < n_cols) {
    for (int r = ry; r < m_rows; r += 16) {
      const uint16_t raw = dz[static_cast<size_t>(r) * ld + col];
      s += (fmt == kOutBf16) ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                             : __half2float(*reinterpret_cast<const __half*>(&raw));
    }
  }
  part[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && col < n_cols) {
    float t = 0.f;
    for (int i = 0; i < 16; ++i) t += part[i][cx];
    out[col] = accumulate ? out[col] + t : t;
  }
}

// ---- moving ignored rows out of the way -----------------------------------------------------------------------
// Stable partition of the row indices: rows whose target is not ignore_index first (in order), the others after them.
// perm[i] = original row of compact row i; *active = number of rows that matter.  One block, ordered.
__global__ void compact_plan_kernel(const long long* target, int n_rows, long long ignore_index, int* perm, int* active) {
  __shared__ int warp_tot[32];
  __shared__ int s_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  // pass 1: how many rows matter
  int cnt = 0;
  for (int i = threadIdx.x; i < n_rows; i += blockDim.x) cnt += target[i] != ignore_index;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) warp_tot[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < n_warps; ++w) t += warp_tot[w];
    s_total = t;
    *active = t;
  }
  __syncthreads();
  const int total = s_total;
  // pass 2: block-wide exclusive scan, one chunk of blockDim.x rows at a time
  int base_valid = 0, base_other = 0;
  for (int c0 = 0; c0 < n_rows; c0 += blockDim.x) {
    const int row = c0 + threadIdx.x;
    const int flag = (row < n_rows) && (target[row] != ignore_index);
    int incl = flag;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    __syncthreads();   // warp_tot is reused
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int warp_base = 0, chunk_valid = 0;
    for (int w = 0; w < n_warps; ++w) {
      const int v = warp_tot[w];
      if (w < warp) warp_base += v;
      chunk_valid += v;
    }
    const int before = warp_base + incl - flag;   // rows that matter before this one inside the chunk
    if (row < n_rows) {
      if (flag) perm[base_valid + before] = row;
      else perm[total + base_other + (threadIdx.x - before)] = row;
    }
    const int chunk_rows = min(static_cast<int>(blockDim.x), n_rows - c0);
    base_valid += chunk_valid;
    base_other += chunk_rows - chunk_valid;
  }
}

// dst row i = src row perm[i] (row_bytes a multiple of 16); targets are permuted alongside
__global__ void gather_rows_kernel(const uint8_t* src, long long src_pitch_bytes, const int* perm, uint8_t* dst,
                                   long long row_bytes, const long long* target, long long* target_out) {
  const int i = blockIdx.x;
  const int from = perm[i];
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(from) * src_pitch_bytes);
  uint4* d = reinterpret_cast<uint4*>(dst + static_cast<size_t>(i) * row_bytes);
  for (long long v = threadIdx.x; v < row_bytes / 16; v += blockDim.x) d[v] = s[v];
  if (threadIdx.x == 0 && target != nullptr) target_out[i] = target[from];
}

// dst row perm[i] = src row i for i < *active, zeros for the rest (row_bytes a multiple of 16)
__global__ void scatter_rows_kernel(const uint8_t* src, const int* perm, const int* active, uint8_t* dst, long long row_bytes) {
  const int i = blockIdx.x;
  const bool live = i < *active;
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(i) * row_bytes);
  uint4* d = reinterpret_cast<uint4*>(dst + static_cast<size_t>(perm[i]) * row_bytes);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (long long v = threadIdx.x; v < row_bytes / 16; v += blockDim.x) d[v] = live ? s[v] : zero;
}

// fp32 -> sum of 16-bit terms: term 0 = round(v), term 1 = round(v - term0), term 2 = round(v - term0 - term1).
// Block b of the destination (columns [b * block_cols, (b+1) * block_cols)) receives term pattern[b]; columns beyond
// `cols` inside a block are zero.
struct SplitPattern { int term[8]; };
__global__ void split_fp32_kernel(const float* src, long long rows, long long cols, long long ld_src, uint16_t* dst,
                                  long long ld_dst, long long block_cols, SplitPattern pat, int n_blocks, int fmt) {
  const long long col = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = blockIdx.y;
  if (row >= rows || col >= block_cols) return;
  float term[3] = {0.f, 0.f, 0.f};
  if (col < cols) {
    float v = src[row * ld_src + col];
#pragma unroll
    for (int t = 0; t < 3; ++t) {
      const float r = (fmt == kOutBf16) ? __bfloat162float(__float2bfloat16_rn(v)) : __half2float(__float2half_rn(v));
      term[t] = r;
      v -= r;
    }
  }
  for (int b = 0; b < n_blocks; ++b) {
    const float t = term[pat.term[b]];
    uint16_t bits;
    if (fmt == kOutBf16) {
      const __nv_bfloat16 h = __float2bfloat16_rn(t);
      bits = *reinterpret_cast<const uint16_t*>(&h);
    } else {
      const __half h = __float2half_rn(t);
      bits = *reinterpret_cast<const uint16_t*>(&h);
    }
    dst[row * ld_dst + b * block_cols + col] = bits;
  }
}

// grad_bias[j] (+)= sum over rows of the 16-bit slab column j; one block per 64 columns, ordered sum
// (rows at and beyond *active_rows, when given, were never written by the sweep and are left out)
__global__ void colsum_kernel(const uint16_t* dz, long long ld, int m_rows, int n_cols, int fmt, float* out,
                              const int* active_rows = nullptr) {
  __shared__ float part[16][64];
  if (active_rows != nullptr) m_rows = min(m_rows, max(0, *active_rows));
  const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;  // 64 x 16
  const int col = blockIdx.x * 64 + cx;
  float s = 0.f;
  if (col < n_cols) {
    for (int r = ry; r < m_rows; r += 16) {
      const uint16_t raw = dz[static_cast<size_t>(r) * ld + col];
      s += (fmt == kOutBf16) ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw))
                             : __half2float(*reinterpret_cast<const __half*>(&raw));
    }
  }
  part[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && col < n_cols) {
    float t = 0.f;
    for (int i = 0; i < 16; ++i) t += part[i][cx];
    out[col] = t;
  }
}

}  // namespace flce
