// Stand-alone cross-entropy on materialised logits (the step beside the fused path when a model keeps its
// logits): two HBM-bound SIMT kernels.  Row statistics come out in the same [6][N] plane format as the fused
// sweep, so the per-row loss, coefficient and reduction kernels are shared with it.
//   ce_stats_kernel : one CTA per row, one read of the row  -> max, sum-exp, target logit, logit sum, arg-max
//   ce_grad_kernel  : one read + one write per element       -> logit gradient (may overwrite the logits)
#pragma once

#include "simt_common.cuh"

namespace flce {

template <typename T>
struct CeElem;
template <>
struct CeElem<float> {
  static constexpr int kVec = 4;
  __device__ static float load(const float* p) { return *p; }
  __device__ static void store(float* p, float v) { *p = v; }
};
template <>
struct CeElem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <>
struct CeElem<__half> {
  static constexpr int kVec = 8;
  __device__ static float load(const __half* p) { return __half2float(*p); }
  __device__ static void store(__half* p, float v) { *p = __float2half_rn(v); }
};

// 16 bytes of elements -> floats
template <typename T>
__device__ __forceinline__ void ce_load_vec(const T* p, float (&v)[CeElem<T>::kVec]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < CeElem<T>::kVec; ++i) v[i] = CeElem<T>::load(e + i);
}
template <typename T>
__device__ __forceinline__ void ce_store_vec(T* p, const float (&v)[CeElem<T>::kVec]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < CeElem<T>::kVec; ++i) CeElem<T>::store(e + i, v[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

struct CeRowState {
  float m, d, ss, best;
  int best_idx;
};

__device__ __forceinline__ void ce_state_init(CeRowState& s) {
  s.m = -INFINITY;
  s.d = 0.f;
  s.ss = 0.f;
  s.best = -INFINITY;
  s.best_idx = 0x7fffffff;
}

// fold one in-range value
__device__ __forceinline__ void ce_state_push(CeRowState& s, float v, float w, int col) {
  if (v > s.best) {  // columns arrive in increasing order within a thread: strictly greater keeps the lowest index
    s.best = v;
    s.best_idx = col;
  }
  s.ss = fmaf(v, w, s.ss);
  const float m_new = fmaxf(s.m, v);
  if (m_new != -INFINITY) {  // a row that is -inf so far contributes nothing yet (and -inf - -inf would be NaN)
    s.d = s.d * ex2_approx((s.m - m_new) * kLog2e) + ex2_approx((v - m_new) * kLog2e);
    s.m = m_new;
  }
}

// fold kVec consecutive in-range values at once: one running-max update and one rescale for the group instead of one per
// element (half the exp2 work of ce_state_push)
template <int kVec>
__device__ __forceinline__ void ce_state_push_vec(CeRowState& s, const float (&v)[kVec], const float* w, int col0) {
  float vmax = v[0];
#pragma unroll
  for (int j = 1; j < kVec; ++j) vmax = fmaxf(vmax, v[j]);
  if (vmax > s.best) {  // strictly greater, and the first position inside the group: the lowest index wins ties
    int idx = kVec - 1;
#pragma unroll
    for (int j = kVec - 2; j >= 0; --j) idx = (v[j] == vmax) ? j : idx;
    s.best = vmax;
    s.best_idx = col0 + idx;
  }
  if (w != nullptr) {
#pragma unroll
    for (int j = 0; j < kVec; ++j) s.ss = fmaf(v[j], w[col0 + j], s.ss);
  } else {
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) a += v[j];
    s.ss += a;
  }
  const float m_new = fmaxf(s.m, vmax);
  if (m_new != -INFINITY) {
    const float ml2 = m_new * kLog2e;
    float e = 0.f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) e += ex2_approx(fmaf(v[j], kLog2e, -ml2));
    s.d = fmaf(s.d, ex2_approx((s.m - m_new) * kLog2e), e);
    s.m = m_new;
  }
}

// merge two partial states of the same row (either may be empty: m = -inf, d = 0)
__device__ __forceinline__ void ce_state_merge(CeRowState& a, const CeRowState& b) {
  if (b.best > a.best || (b.best == a.best && b.best_idx < a.best_idx)) {
    a.best = b.best;
    a.best_idx = b.best_idx;
  }
  a.ss += b.ss;
  const float m_new = fmaxf(a.m, b.m);
  if (m_new != -INFINITY) {
    a.d = a.d * ex2_approx((a.m - m_new) * kLog2e) + b.d * ex2_approx((b.m - m_new) * kLog2e);
    a.m = m_new;
  }
}

constexpr int kCeThreads = 256;
constexpr int kCeGradUnroll = 4;   // vectors per thread of ce_grad_kernel

template <typename T, bool kVectorised>
__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const T* logits, long long ld, int n_rows, int n_cols, const long long* target, const float* col_weight,
                float softcap, float inv_softcap, float* rowstats) {
  __shared__ CeRowState warp_state[kCeThreads / 32];
  const int row = blockIdx.x;
  if (row >= n_rows) return;
  const T* x = logits + static_cast<size_t>(row) * ld;
  CeRowState st;
  ce_state_init(st);
  constexpr int kVec = CeElem<T>::kVec;
  int tail_begin = 0;
  if constexpr (kVectorised) {
    const int n_vec = n_cols / kVec;
    tail_begin = n_vec * kVec;
    // four 16-byte loads per thread in flight before any of them is used: one CTA per row has to keep HBM busy
    constexpr int kUnroll = 4;
    for (int i0 = threadIdx.x; i0 < n_vec; i0 += kCeThreads * kUnroll) {
      uint4 raw[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int i = i0 + u * kCeThreads;
        if (i < n_vec) raw[u] = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(i) * kVec);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int i = i0 + u * kCeThreads;
        if (i >= n_vec) break;
        const T* e = reinterpret_cast<const T*>(&raw[u]);
        float v[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          v[j] = CeElem<T>::load(e + j);
          if (softcap > 0.f) v[j] = softcap * tanh_accurate(v[j] * inv_softcap);
        }
        ce_state_push_vec<kVec>(st, v, col_weight, i * kVec);
      }
    }
  }
  for (int col = tail_begin + threadIdx.x; col < n_cols; col += kCeThreads) {
    float s = CeElem<T>::load(x + col);
    if (softcap > 0.f) s = softcap * tanh_accurate(s * inv_softcap);
    ce_state_push(st, s, col_weight != nullptr ? col_weight[col] : 1.f, col);
  }
  // warp tree, then one warp over the per-warp results: a fixed order, so the result is run-to-run identical
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    CeRowState other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.d = __shfl_xor_sync(0xffffffffu, st.d, o);
    other.ss = __shfl_xor_sync(0xffffffffu, st.ss, o);
    other.best = __shfl_xor_sync(0xffffffffu, st.best, o);
    other.best_idx = __shfl_xor_sync(0xffffffffu, st.best_idx, o);
    ce_state_merge(st, other);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) warp_state[warp] = st;
  __syncthreads();
  if (warp == 0) {
    CeRowState acc;
    ce_state_init(acc);
    if (lane < kCeThreads / 32) acc = warp_state[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      CeRowState other;
      other.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
      other.d = __shfl_xor_sync(0xffffffffu, acc.d, o);
      other.ss = __shfl_xor_sync(0xffffffffu, acc.ss, o);
      other.best = __shfl_xor_sync(0xffffffffu, acc.best, o);
      other.best_idx = __shfl_xor_sync(0xffffffffu, acc.best_idx, o);
      ce_state_merge(acc, other);
    }
    if (lane == 0) {
      const size_t n = static_cast<size_t>(n_rows);
      float xy = 0.f;
      const long long t = target[row];
      if (t >= 0 && t < n_cols) {
        xy = CeElem<T>::load(x + t);
        if (softcap > 0.f) xy = softcap * tanh_accurate(xy * inv_softcap);
      }
      rowstats[0 * n + row] = acc.m;
      rowstats[1 * n + row] = acc.d;
      rowstats[2 * n + row] = xy;
      rowstats[3 * n + row] = acc.ss;
      rowstats[4 * n + row] = acc.best;
      reinterpret_cast<int*>(rowstats)[5 * n + row] = acc.best_idx == 0x7fffffff ? 0 : acc.best_idx;
    }
  }
}

// grad[r][j] = (exp(s - lse_r) * c1_r - c2_r * w_j - c3_r * [j == target_r]) * (1 - tanh^2(z / softcap)); grad may alias logits
template <typename T, bool kVectorised>
__global__ void __launch_bounds__(kCeThreads)
ce_grad_kernel(const T* logits, long long ld, T* grad, long long ld_grad, int n_rows, int n_cols, const long long* target,
               const float* col_weight, float softcap, float inv_softcap, const float* lse, const float* c1,
               const float* c2, const float* c3) {
  const int row = blockIdx.x;   // rows on x: no 65535 limit
  if (row >= n_rows) return;
  constexpr int kVec = kVectorised ? CeElem<T>::kVec : 1;
  const float l2 = lse[row] * kLog2e, a = c1[row], b = c2[row], c = c3[row];
  const long long t = target[row];
  const T* xrow = logits + static_cast<size_t>(row) * ld;
  T* grow = grad + static_cast<size_t>(row) * ld_grad;
  auto one = [&](float z, int col) {
    float s = z, chain = 1.f;
    if (softcap > 0.f) {
      const float th = tanh_accurate(z * inv_softcap);
      s = softcap * th;
      chain = fmaf(-th, th, 1.f);
    }
    const float wj = col_weight != nullptr ? col_weight[col] : 1.f;
    float v = fmaf(ex2_approx(fmaf(s, kLog2e, -l2)), a, -b * wj);
    if (static_cast<long long>(col) == t) v -= c;
    return v * chain;
  };
  // a block covers kCeGradUnroll * kCeThreads vectors of one row; all of a thread's loads are issued before the math
  const int base = blockIdx.y * (kCeThreads * kCeGradUnroll) * kVec + threadIdx.x * kVec;
  if constexpr (kVectorised) {
    uint4 raw[kCeGradUnroll];
#pragma unroll
    for (int u = 0; u < kCeGradUnroll; ++u) {
      const int col0 = base + u * kCeThreads * kVec;
      if (col0 + kVec <= n_cols) raw[u] = *reinterpret_cast<const uint4*>(xrow + col0);
    }
#pragma unroll
    for (int u = 0; u < kCeGradUnroll; ++u) {
      const int col0 = base + u * kCeThreads * kVec;
      if (col0 >= n_cols) break;
      if (col0 + kVec <= n_cols) {
        const T* e = reinterpret_cast<const T*>(&raw[u]);
        float v[CeElem<T>::kVec];
#pragma unroll
        for (int j = 0; j < CeElem<T>::kVec; ++j) v[j] = one(CeElem<T>::load(e + j), col0 + j);
        ce_store_vec<T>(grow + col0, v);
      } else {
        for (int j = 0; col0 + j < n_cols; ++j) CeElem<T>::store(grow + col0 + j, one(CeElem<T>::load(xrow + col0 + j), col0 + j));
      }
    }
  } else {
#pragma unroll
    for (int u = 0; u < kCeGradUnroll; ++u) {
      const int col0 = base + u * kCeThreads;
      if (col0 < n_cols) CeElem<T>::store(grow + col0, one(CeElem<T>::load(xrow + col0), col0));
    }
  }
}

}  // namespace flce
