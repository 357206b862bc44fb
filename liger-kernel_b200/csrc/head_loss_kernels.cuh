// Row kernels of the two sibling losses of the fused linear cross-entropy path, working on a token chunk's logits
// that a tensor-core GEMM of this library has just written (16-bit or fp32 slab, row pitch `ld` elements):
//
//   scaled_ce_rows_kernel : per token, at temperature T: nll = lse(s) - s_y and entropy = lse(s) - sum_j p_j s_j
//   scaled_ce_grad_kernel : in place, d z_j = [g_nll (p_j - [j = y]) - g_ent p_j (log p_j + entropy)] / T
//   jsd_rows_kernel       : generalised Jensen-Shannon divergence between a student row and a teacher row; the
//                           student slab is overwritten by the gradient with respect to the student's logits
//
// One CTA per row for the reductions (fixed-order trees: run-to-run identical), 16-byte accesses when the slab allows.
// The JSD kernel keeps the rows in flight within L2 (see there).
// SIMT only: this header also compiles for the host emulation the CPU tests use.
#pragma once

#include "ce_kernels.cuh"

namespace flce {

// ---- online (max, sum exp, sum exp * value) ---------------------------------------------------------------------
struct EntropyState {
  float m, d, t;
};

__device__ __forceinline__ void ent_init(EntropyState& s) {
  s.m = -INFINITY;
  s.d = 0.f;
  s.t = 0.f;
}

__device__ __forceinline__ void ent_push(EntropyState& s, float v) {
  if (v == -INFINITY) return;  // a masked class: probability 0, and 0 * -inf must not reach the sums
  const float m_new = fmaxf(s.m, v);
  const float keep = ex2_approx((s.m - m_new) * kLog2e);  // 0 when the state was empty
  const float e = ex2_approx((v - m_new) * kLog2e);
  s.d = fmaf(s.d, keep, e);
  s.t = fmaf(s.t, keep, e * v);
  s.m = m_new;
}

__device__ __forceinline__ void ent_merge(EntropyState& a, const EntropyState& b) {
  const float m_new = fmaxf(a.m, b.m);
  if (m_new == -INFINITY) return;
  const float ka = ex2_approx((a.m - m_new) * kLog2e), kb = ex2_approx((b.m - m_new) * kLog2e);
  a.d = a.d * ka + b.d * kb;
  a.t = a.t * ka + b.t * kb;
  a.m = m_new;
}

template <int kThreads = kCeThreads>
__device__ __forceinline__ EntropyState ent_block_reduce(EntropyState st, EntropyState* warp_state) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    EntropyState other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.d = __shfl_xor_sync(0xffffffffu, st.d, o);
    other.t = __shfl_xor_sync(0xffffffffu, st.t, o);
    ent_merge(st, other);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // warp_state may still be read by the previous reduction
  if (lane == 0) warp_state[warp] = st;
  __syncthreads();
  EntropyState acc;
  ent_init(acc);
  if (lane < kThreads / 32) acc = warp_state[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    EntropyState other;
    other.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
    other.d = __shfl_xor_sync(0xffffffffu, acc.d, o);
    other.t = __shfl_xor_sync(0xffffffffu, acc.t, o);
    ent_merge(acc, other);
  }
  return acc;  // every warp computes the same total from the same values in the same order
}

// sum of two floats per thread over the block, fixed order; result valid in every thread
template <int kThreads = kCeThreads>
__device__ __forceinline__ float2 block_sum2(float a, float b, float2* warp_part) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) warp_part[warp] = make_float2(a, b);
  __syncthreads();
  float2 r = make_float2(0.f, 0.f);
  if (lane < kThreads / 32) r = warp_part[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    r.x += __shfl_xor_sync(0xffffffffu, r.x, o);
    r.y += __shfl_xor_sync(0xffffffffu, r.y, o);
  }
  return r;
}

// visit every element of a row once: f(value, column); 16-byte loads over the aligned body
template <typename T, bool kVectorised, int kThreads = kCeThreads, typename F>
__device__ __forceinline__ void for_each_in_row(const T* x, int n_cols, F&& f) {
  constexpr int kVec = CeElem<T>::kVec;
  int tail_begin = 0;
  if constexpr (kVectorised) {
    const int n_vec = n_cols / kVec;
    tail_begin = n_vec * kVec;
    for (int i = threadIdx.x; i < n_vec; i += kThreads) {
      float v[kVec];
      ce_load_vec<T>(x + i * kVec, v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) f(v[j], i * kVec + j);
    }
  }
  for (int col = tail_begin + threadIdx.x; col < n_cols; col += kThreads) f(CeElem<T>::load(x + col), col);
}

// ---- scaled cross-entropy ------------------------------------------------------------------------------------------
// nll / entropy are 0 on ignored rows; lse is written for every row.
template <typename T, bool kVectorised>
__global__ void __launch_bounds__(kCeThreads)
scaled_ce_rows_kernel(const T* logits, long long ld, int n_rows, int n_cols, const long long* target, long long ignore_index,
                      float inv_temperature, float* nll, float* entropy, float* lse_out) {
  __shared__ EntropyState warp_state[kCeThreads / 32];
  const int row = blockIdx.x;
  if (row >= n_rows) return;
  const T* x = logits + static_cast<size_t>(row) * ld;
  EntropyState st;
  ent_init(st);
  for_each_in_row<T, kVectorised>(x, n_cols, [&](float z, int) { ent_push(st, z * inv_temperature); });
  const EntropyState acc = ent_block_reduce(st, warp_state);
  if (threadIdx.x == 0) {
    const float lse = acc.m + logf(acc.d);
    const long long t = target[row];
    float out_nll = 0.f, out_ent = 0.f;
    if (t != ignore_index) {
      const float sy = (t >= 0 && t < n_cols) ? CeElem<T>::load(x + t) * inv_temperature : 0.f;
      out_nll = lse - sy;
      out_ent = lse - acc.t / acc.d;
    }
    nll[row] = out_nll;
    entropy[row] = out_ent;
    lse_out[row] = lse;
  }
}

// in place over the chunk's logits; rows on grid.x
template <typename T, bool kVectorised>
__global__ void __launch_bounds__(kCeThreads)
scaled_ce_grad_kernel(T* logits, long long ld, int n_rows, int n_cols, const long long* target, long long ignore_index,
                      float inv_temperature, const float* lse, const float* entropy, const float* grad_nll,
                      const float* grad_entropy) {
  const int row = blockIdx.x;
  if (row >= n_rows) return;
  constexpr int kVec = kVectorised ? CeElem<T>::kVec : 1;
  const int col0 = (blockIdx.y * kCeThreads + threadIdx.x) * kVec;
  if (col0 >= n_cols) return;
  const long long t = target[row];
  const bool live = t != ignore_index;
  const float g_nll = (live && grad_nll != nullptr) ? grad_nll[row] : 0.f;
  const float g_ent = (live && grad_entropy != nullptr) ? grad_entropy[row] : 0.f;
  const float row_lse = lse[row], h = entropy[row];
  T* x = logits + static_cast<size_t>(row) * ld + col0;
  auto one = [&](float z, int col) {
    const float s = z * inv_temperature;
    const float logp = s - row_lse;
    const float p = ex2_approx(logp * kLog2e);
    float v = p * (g_nll - g_ent * (logp + h));
    if (static_cast<long long>(col) == t) v -= g_nll;
    return (live && z != -INFINITY) ? v * inv_temperature : 0.f;
  };
  if constexpr (kVectorised) {
    if (col0 + kVec <= n_cols) {
      float v[CeElem<T>::kVec];
      ce_load_vec<T>(x, v);
#pragma unroll
      for (int j = 0; j < CeElem<T>::kVec; ++j) v[j] = one(v[j], col0 + j);
      ce_store_vec<T>(x, v);
      return;
    }
    for (int j = 0; col0 + j < n_cols; ++j) CeElem<T>::store(x + j, one(CeElem<T>::load(x + j), col0 + j));
  } else {
    CeElem<T>::store(x, one(CeElem<T>::load(x), col0));
  }
}

// per-(row, tile) partials of EntropyStatsEpilogue -> per-row nll, entropy (0 on ignored rows) and lse
__global__ void scaled_ce_merge_kernel(int m_rows, int n_tiles, const float* pmax, const float* psum, const float* pts,
                                       const float* target_logit, const long long* target, long long ignore_index, float* nll,
                                       float* entropy, float* lse_out) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= m_rows) return;
  float m = -INFINITY;
  for (int i = 0; i < n_tiles; ++i) m = fmaxf(m, pmax[static_cast<size_t>(i) * m_rows + row]);
  float d = 0.f, t = 0.f;
  for (int i = 0; i < n_tiles; ++i) {
    const size_t o = static_cast<size_t>(i) * m_rows + row;
    const float k = expf(pmax[o] - m);
    d = fmaf(psum[o], k, d);
    t = fmaf(pts[o], k, t);
  }
  const float lse = m + logf(d);
  const bool live = target[row] != ignore_index;
  nll[row] = live ? lse - target_logit[row] : 0.f;
  entropy[row] = live ? lse - t / d : 0.f;
  lse_out[row] = lse;
}

// ---- generalised Jensen-Shannon divergence -----------------------------------------------------------------------
// X = log Q = s - lse_s, Y = log P = t - lse_t (both at the temperature).  Returns the element's loss term and the
// derivative with respect to X.  beta == 0: forward KL, beta == 1: reverse KL.
__device__ __forceinline__ void jsd_terms(float X, float Y, float beta, float& loss, float& dX, float& Q) {
  Q = ex2_approx(X * kLog2e);
  const float P = ex2_approx(Y * kLog2e);
  if (beta == 0.f) {
    loss = (P > 0.f) ? P * (Y - X) : 0.f;
    dX = -P;
  } else if (beta == 1.f) {
    loss = (Q > 0.f) ? Q * (X - Y) : 0.f;
    dX = loss + Q;
  } else {
    const float bP = beta * P, bQ = (1.f - beta) * Q;
    const float M = bP + bQ;
    if (M >= 1.17549435e-38f) {   // below the smallest normal the term is worth less than 1e-36 (and lg2.approx reads a subnormal as 0)
      const float log_m = ln_approx(M);   // M in [2^-126, 1]: the approximate logarithm is good to about 2e-7 absolute here
      loss = (bP > 0.f ? bP * Y : 0.f) + (bQ > 0.f ? bQ * X : 0.f) - M * log_m;
      dX = (bQ > 0.f) ? bQ * (X - log_m) : 0.f;
    } else {
      loss = 0.f;
      dX = 0.f;
    }
  }
}

// A CTA of kJsdThreads threads per SM walks over the tokens (row = blockIdx.x, += gridDim.x): one student row and one teacher
// row of a 128 k vocabulary are 513 KB in 16-bit, so 148 rows in flight fit the 126 MB L2 and the second and third sweep of a
// row are served from it; with one small CTA per row several times as many rows would be resident and every sweep would go to
// HBM.  `count` (device, may be null) holds the number of tokens that matter; with null, `fixed_count` is used.
// loss_rows[row] receives the token's share of the loss (already divided by the count); the student's row is overwritten with
// d loss / d (student logits), zeros when the token's label is ignore_index.
#ifndef FLCE_JSD_THREADS
#define FLCE_JSD_THREADS 1024   // the host emulation of the CPU tests builds this kernel with fewer threads to stay fast
#endif
constexpr int kJsdThreads = FLCE_JSD_THREADS;

template <typename T, bool kVectorised>
__global__ void __launch_bounds__(kJsdThreads, 1)
jsd_rows_kernel(T* student, long long ld_s, const T* teacher, long long ld_t, int n_rows, int n_cols, const long long* labels,
                long long ignore_index, float beta, float inv_temperature, const float* count, float fixed_count,
                float* loss_rows) {
  __shared__ EntropyState warp_state[kJsdThreads / 32];
  __shared__ float2 warp_part[kJsdThreads / 32];
  constexpr int kVec = CeElem<T>::kVec;
  const float n_live = count != nullptr ? *count : fixed_count;
  const float scale = n_live > 0.f ? 1.f / n_live : 0.f;
  const float out_scale = scale * inv_temperature;
  for (int row = blockIdx.x; row < n_rows; row += gridDim.x) {   // uniform per CTA: the barriers below are reached by all threads
    T* xs = student + static_cast<size_t>(row) * ld_s;
    const T* xt = teacher + static_cast<size_t>(row) * ld_t;
    if (labels != nullptr && labels[row] == ignore_index) {
      for (int col = threadIdx.x; col < n_cols; col += kJsdThreads) CeElem<T>::store(xs + col, 0.f);
      if (threadIdx.x == 0) loss_rows[row] = 0.f;
      continue;
    }
    // sweep 1: both log-normalisers
    EntropyState a, b;
    ent_init(a);
    ent_init(b);
    const int n_vec = kVectorised ? n_cols / kVec : 0;
    for (int i = threadIdx.x; i < n_vec; i += kJsdThreads) {   // both rows in one loop: two independent loads in flight
      float vs[kVec], vt[kVec];
      ce_load_vec<T>(xs + i * kVec, vs);
      ce_load_vec<T>(xt + i * kVec, vt);
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        ent_push(a, vs[j] * inv_temperature);
        ent_push(b, vt[j] * inv_temperature);
      }
    }
    for (int col = n_vec * kVec + threadIdx.x; col < n_cols; col += kJsdThreads) {
      ent_push(a, CeElem<T>::load(xs + col) * inv_temperature);
      ent_push(b, CeElem<T>::load(xt + col) * inv_temperature);
    }
    a = ent_block_reduce<kJsdThreads>(a, warp_state);
    b = ent_block_reduce<kJsdThreads>(b, warp_state);
    const float lse_s = a.m + logf(a.d), lse_t = b.m + logf(b.d);
    // sweep 2: the token's loss and sum_k dX_k
    float loss_acc = 0.f, dx_acc = 0.f;
    for (int i = threadIdx.x; i < n_vec; i += kJsdThreads) {
      float vs[kVec], vt[kVec];
      ce_load_vec<T>(xs + i * kVec, vs);
      ce_load_vec<T>(xt + i * kVec, vt);
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        float l, dx, q;
        jsd_terms(vs[j] * inv_temperature - lse_s, vt[j] * inv_temperature - lse_t, beta, l, dx, q);
        loss_acc += l;
        dx_acc += dx;
      }
    }
    for (int col = n_vec * kVec + threadIdx.x; col < n_cols; col += kJsdThreads) {
      float l, dx, q;
      jsd_terms(CeElem<T>::load(xs + col) * inv_temperature - lse_s, CeElem<T>::load(xt + col) * inv_temperature - lse_t, beta, l,
                dx, q);
      loss_acc += l;
      dx_acc += dx;
    }
    const float2 tot = block_sum2<kJsdThreads>(loss_acc, dx_acc, warp_part);
    if (threadIdx.x == 0) loss_rows[row] = tot.x * scale;
    // sweep 3: d logits = (dX - Q * sum dX) * scale / T, over the student's row
    for (int i = threadIdx.x; i < n_vec; i += kJsdThreads) {
      float vs[kVec], vt[kVec];
      ce_load_vec<T>(xs + i * kVec, vs);
      ce_load_vec<T>(xt + i * kVec, vt);
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        float l, dx, q;
        jsd_terms(vs[j] * inv_temperature - lse_s, vt[j] * inv_temperature - lse_t, beta, l, dx, q);
        vs[j] = (dx - q * tot.y) * out_scale;
      }
      ce_store_vec<T>(xs + i * kVec, vs);
    }
    for (int col = n_vec * kVec + threadIdx.x; col < n_cols; col += kJsdThreads) {
      float l, dx, q;
      jsd_terms(CeElem<T>::load(xs + col) * inv_temperature - lse_s, CeElem<T>::load(xt + col) * inv_temperature - lse_t, beta, l,
                dx, q);
      CeElem<T>::store(xs + col, (dx - q * tot.y) * out_scale);
    }
  }
}

}  // namespace flce
