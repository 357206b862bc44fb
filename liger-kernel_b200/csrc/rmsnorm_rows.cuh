// The caller in front of the fused path: the final RMSNorm of a decoder feeds `hidden_states` into the head
// (src/liger_kernel/ops/rms_norm.py:59-139 forward, :143-235 backward of the reference).  Here it is folded into the two
// row moves the fused path makes anyway: the gather that puts the rows that matter first (the tensor-core sweeps read the
// result through TMA) normalises on the way, and the scatter that returns grad_input to token order applies the norm's
// backward on the way.  The normalised [BT, H] tensor never exists in token order and is neither written nor re-read by a
// separate kernel.
//
//   y_j = x_j * rstd * (offset + g_j),  rstd = rsqrt(mean(x^2) + eps)
//   casting mode 0 ("llama"): x * rstd is rounded to the input dtype before it meets the weight;
//   casting mode 1 ("gemma"): everything in fp32, one rounding at the end.
//   dx = rstd * m - rstd^3 / H * sum(m * x) * x,  m = dy * (offset + g);   dg = sum over rows of dy * (x * rstd)
#pragma once

#include "ce_kernels.cuh"
#include "simt_common.cuh"

namespace flce {

constexpr int kRmsThreads = 256;      // the gather; the backward uses 256 or 512
constexpr int kRmsMaxVecs = 4;        // 16-byte vectors of a row per thread in the backward: rows of up to 512 * 4 * 8 = 16384
                                      // 16-bit elements
constexpr int kRmsModeLlama = 0;
constexpr int kRmsModeGemma = 1;

// sum over the block, returned to every thread; scratch: 32 floats of shared memory; two barriers
__device__ __forceinline__ float rms_block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                      // the previous use of scratch has been read
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = 0.f;
  for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) r += scratch[w];   // the same order in every thread
  return r;
}

// dst row i = rmsnorm(src row perm[i]) (perm == nullptr: row i), rstd_out[i] = its 1 / rms, targets permuted alongside.
// One block per destination row; the row is read twice (the second time from L1 / L2).
template <typename T>
__global__ void __launch_bounds__(kRmsThreads)
rmsnorm_gather_rows_kernel(const T* src, long long src_pitch, const int* perm, T* dst, long long dst_pitch, int hidden,
                           const T* gamma, float eps, float offset, int mode, float* rstd_out, const long long* target,
                           long long* target_out) {
  __shared__ float scratch[32];
  constexpr int kVec = CeElem<T>::kVec;
  const int i = blockIdx.x;
  const int from = perm != nullptr ? perm[i] : i;
  const T* x = src + static_cast<size_t>(from) * src_pitch;
  T* y = dst + static_cast<size_t>(i) * dst_pitch;
  const int n_vec = hidden / kVec;
  float ss = 0.f;
  for (int v = threadIdx.x; v < n_vec; v += kRmsThreads) {
    float e[kVec];
    ce_load_vec<T>(x + v * kVec, e);
#pragma unroll
    for (int j = 0; j < kVec; ++j) ss = fmaf(e[j], e[j], ss);
  }
  const float rstd = 1.f / sqrtf(rms_block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
  for (int v = threadIdx.x; v < n_vec; v += kRmsThreads) {
    float e[kVec], g[kVec], o[kVec];
    ce_load_vec<T>(x + v * kVec, e);
    ce_load_vec<T>(gamma + v * kVec, g);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      float xs = e[j] * rstd;
      if (mode == kRmsModeLlama) {          // rounded to the input dtype before the weight
        T r;
        CeElem<T>::store(&r, xs);
        xs = CeElem<T>::load(&r);
      }
      o[j] = xs * (offset + g[j]);
    }
    ce_store_vec<T>(y + v * kVec, o);
  }
  if (threadIdx.x == 0) {
    rstd_out[i] = rstd;
    if (target != nullptr) target_out[i] = target[from];
  }
}

// grad_hidden row perm[i] = RMSNorm backward of grad_normed row i for i < *active, zeros for the rest;
// dgamma_partial[block][:] = this block's share of sum_i dy_i * (x_i * rstd_i).  A fixed grid of blocks strides over the
// rows, each thread keeps the partial weight gradient of its own columns in registers.
template <typename T, int kVecs>
__global__ void __launch_bounds__(512)
rmsnorm_backward_scatter_kernel(const T* grad_normed, long long g_pitch, const T* src, long long src_pitch, const T* gamma,
                                const float* rstd, const int* perm, const int* active, int n_rows, int hidden, float offset,
                                int mode, T* grad_hidden, long long gx_pitch, float* dgamma_partial) {
  __shared__ float scratch[32];
  constexpr int kVec = CeElem<T>::kVec;
  const int n_vec = hidden / kVec;
  const int threads = static_cast<int>(blockDim.x);
  const int live = active != nullptr ? *active : n_rows;
  float dg[kVecs][kVec];
#pragma unroll
  for (int u = 0; u < kVecs; ++u) {
#pragma unroll
    for (int j = 0; j < kVec; ++j) dg[u][j] = 0.f;
  }
  for (int i = blockIdx.x; i < n_rows; i += gridDim.x) {
    const int to = perm != nullptr ? perm[i] : i;
    T* gx = grad_hidden + static_cast<size_t>(to) * gx_pitch;
    if (i >= live) {                    // uniform across the block
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      for (int v = threadIdx.x; v < n_vec; v += threads) reinterpret_cast<uint4*>(gx)[v] = zero;
      continue;
    }
    const T* dy = grad_normed + static_cast<size_t>(i) * g_pitch;
    const T* x = src + static_cast<size_t>(to) * src_pitch;
    const float r = rstd[i];
    float m[kVecs][kVec], xv[kVecs][kVec];
    float dot = 0.f;
#pragma unroll
    for (int u = 0; u < kVecs; ++u) {
      const int v = threadIdx.x + u * threads;
      if (v < n_vec) {
        float d[kVec], g[kVec];
        ce_load_vec<T>(dy + v * kVec, d);
        ce_load_vec<T>(x + v * kVec, xv[u]);
        ce_load_vec<T>(gamma + v * kVec, g);        // the same few KB for every row: stays in L1
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          m[u][j] = d[j] * (offset + g[j]);
          dot = fmaf(m[u][j], xv[u][j], dot);
          float xs = xv[u][j] * r;
          if (mode == kRmsModeLlama) {
            T q;
            CeElem<T>::store(&q, xs);
            xs = CeElem<T>::load(&q);
          }
          dg[u][j] = fmaf(d[j], xs, dg[u][j]);
        }
      }
    }
    const float total = rms_block_sum(dot, scratch);
    const float c = -r * r * r * total / static_cast<float>(hidden);
#pragma unroll
    for (int u = 0; u < kVecs; ++u) {
      const int v = threadIdx.x + u * threads;
      if (v < n_vec) {
        float o[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) o[j] = fmaf(c, xv[u][j], r * m[u][j]);
        ce_store_vec<T>(gx + v * kVec, o);
      }
    }
  }
  float* mine = dgamma_partial + static_cast<size_t>(blockIdx.x) * hidden;
#pragma unroll
  for (int u = 0; u < kVecs; ++u) {
    const int v = threadIdx.x + u * threads;
    if (v < n_vec) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) mine[v * kVec + j] = dg[u][j];
    }
  }
}

// dgamma[c] = sum over the blocks' partials, in block order
__global__ void rmsnorm_dgamma_reduce_kernel(const float* partial, int n_blocks, int hidden, float* dgamma) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= hidden) return;
  float s = 0.f;
  for (int b = 0; b < n_blocks; ++b) s += partial[static_cast<size_t>(b) * hidden + c];
  dgamma[c] = s;
}

}  // namespace flce
