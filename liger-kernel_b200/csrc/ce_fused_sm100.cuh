// Stand-alone cross-entropy with the gradient formed in the same launch (what the reference's kernel does: its forward
// leaves the logit gradient in the logits buffer, src/liger_kernel/ops/cross_entropy.py:41-336), laid out for B200:
//
// * a row of logits is held in the shared memory of a thread-block cluster while it is needed more than once: 1, 2, 4 or
//   8 CTAs each keep one contiguous slice, so HBM sees every logit once on the way in and every gradient once on the way
//   out (2 * n_rows * vocab * sizeof(element) bytes; the two-kernel form moves 3 *);
// * one cluster works on one row, and several CTAs share an SM, so that one row's fetch, another's arithmetic and a third's
//   store overlap.  Each warp owns one piece of its CTA's slice: lane 0 fetches it with one untiled bulk copy that
//   completes on the warp's own mbarrier and hands it back with one bulk store, so a CTA has its whole slice in flight at
//   once without any thread holding load registers, and the only CTA-wide meeting points are the reductions of the row
//   statistics;
// * the per-slice statistics (maximum, sum of exponentials, logit sum, arg-max) meet through distributed shared memory:
//   every CTA writes its five numbers into every peer, one cluster barrier, every CTA merges them in rank order (so all
//   of them hold bit-identical row statistics), computes the row's loss terms and gradient coefficients itself and
//   rewrites its slice in place.
//
// Requirements checked by the launcher: vocab a multiple of the 16-byte vector, row pitches and base addresses 16-byte
// aligned, slice of at most kCeFusedMaxSliceBytes.  Rows whose target is ignore_index are not read: their gradient is zero.
#pragma once

#include "ce_kernels.cuh"
#include "ptx_sm100.cuh"
#include "row_kernels.cuh"

namespace flce {

constexpr int kCeFusedMaxCluster = 8;
constexpr int kCeFusedSmallSliceBytes = 72 * 1024;    // three CTAs per SM: one fetches while another computes or stores
constexpr int kCeFusedMaxSliceBytes = 200 * 1024;     // one CTA per SM
constexpr int kDevTimeoutCeFused = 7;                  // device status when a piece never arrived

struct CeFusedOut {
  float* rowstats;          // [6][n_rows]
  float* lse;
  float* target_prob;
  float* loss_rows;
  float* z_rows;
  float* correct_rows;
  long long* predicted;
};

__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}

// store 32 bits into the same shared-memory offset of CTA `cta` of this cluster
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t local_addr, uint32_t cta, uint32_t v) {
  asm volatile(
      "{\n\t"
      ".reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "st.shared::cluster.u32 [remote], %2;\n\t"
      "}\n" ::"r"(local_addr),
      "r"(cta), "r"(v)
      : "memory");
}

// kStoreExp (no soft-cap): the first pass over shared memory only finds the slice's maximum and arg-max; the second
// forms e = exp(z - slice maximum) once per logit, sums it and leaves e in the logit's place; the last turns e into the
// gradient with one multiply-add, e * (c1 * exp(slice maximum - lse)) - c2 * w: one exponential per logit instead of two.
// The target's own entry is recomputed from the fp32 target logit (it is a small difference of large terms).  Without
// kStoreExp the statistics pass is the online form of ce_stats_kernel and the gradient pass recomputes the exponential.
// One cluster per row, kWarps warps per CTA; several CTAs share an SM, so that one row's fetch, another's arithmetic and a
// third's store overlap.
template <typename T, bool kStoreExp, int kWarps>
__global__ void __launch_bounds__(kWarps * 32)
ce_fused_kernel(const T* logits, long long ld, T* grad, long long ld_grad, int n_rows, int n_cols, int slice_vecs,
                const long long* target, const float* col_weight, float softcap, float inv_softcap, RowMath rm,
                const float* norm, CeFusedOut out, int* status) {
  constexpr int kVec = CeElem<T>::kVec;
  static_assert(kWarps <= 32, "the cross-warp reductions read one warp result per lane");
  extern __shared__ __align__(128) uint8_t ce_fused_smem[];
  __shared__ __align__(8) uint64_t piece_bar[kWarps];
  __shared__ CeRowState warp_state[kWarps];
  __shared__ CeRowState peer_state[kCeFusedMaxCluster];
  __shared__ float warp_max[kWarps];
  __shared__ int warp_argmax[kWarps];

  const uint32_t n_ctas = cluster_nctarank();
  const uint32_t rank = cluster_ctarank();
  const int row = static_cast<int>(blockIdx.x / n_ctas);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = target[row];
  const T* xrow = logits + static_cast<size_t>(row) * ld;
  T* grow = grad + static_cast<size_t>(row) * ld_grad;

  // this CTA's slice and this warp's piece of it, in 16-byte vectors of the row
  const int n_vec = n_cols / kVec;
  const int slice_begin = min(n_vec, static_cast<int>(rank) * slice_vecs);
  const int slice_end = min(n_vec, slice_begin + slice_vecs);
  const int piece_vecs = (slice_vecs + kWarps - 1) / kWarps;
  const int piece_begin = min(slice_end, slice_begin + warp * piece_vecs);
  const int piece_end = min(slice_end, piece_begin + piece_vecs);
  const int my_vecs = piece_end - piece_begin;
  const uint32_t my_bytes = static_cast<uint32_t>(my_vecs) * 16u;
  uint4* piece_smem = reinterpret_cast<uint4*>(ce_fused_smem) + (piece_begin - slice_begin);

  if (t == rm.ignore_index) {
    // uniform across the cluster: nothing to read, the gradient of the row is zero
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int i = piece_begin + lane; i < piece_end; i += 32) reinterpret_cast<uint4*>(grow)[i] = zero;
    if (rank == 0 && threadIdx.x == 0) {
      const size_t n = static_cast<size_t>(n_rows);
      out.rowstats[0 * n + row] = 0.f;
      out.rowstats[1 * n + row] = 1.f;
      out.rowstats[2 * n + row] = 0.f;
      out.rowstats[3 * n + row] = 0.f;
      out.rowstats[4 * n + row] = 0.f;
      reinterpret_cast<int*>(out.rowstats)[5 * n + row] = 0;
      finalize_row(row, rm, t, col_weight, 0.f, 1.f, 0.f, 0.f, 0, norm, out.lse, out.target_prob, out.loss_rows, out.z_rows,
                   out.correct_rows, out.predicted);
    }
    return;
  }

  // ---- fetch: one bulk copy per warp
  const uint32_t bar = smem_u32(&piece_bar[warp]);
  if (lane == 0) {
    mbar_init(bar, 1);
    fence_barrier_init();
    if (my_vecs > 0) {
      mbar_arrive_expect_tx(bar, my_bytes);
      bulk_load_1d(smem_u32(piece_smem), reinterpret_cast<const uint4*>(xrow) + piece_begin, my_bytes, bar);
    }
  }
  // everything the row's arithmetic needs from global memory is requested while the copy is in flight
  float xy = 0.f;
  if (t >= 0 && t < n_cols) {
    xy = CeElem<T>::load(xrow + t);
    if (softcap > 0.f) xy = softcap * tanh_accurate(xy * inv_softcap);
  }
  const float norm_here[4] = {norm[0], norm[1], norm[2], 0.f};
  __syncwarp();
  bool arrived = true;
  if (my_vecs > 0) {
    // bounded: a copy that never completes ends as an error code, not as a hung GPU
    arrived = mbar_try_wait(bar, 0);
    uint64_t t0 = 0;
    for (uint32_t spin = 1; !arrived; ++spin) {
      arrived = mbar_try_wait(bar, 0);
      if (!arrived && (spin & 0x3FFu) == 0) {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > kWaitLimitNs) break;
      }
    }
    arrived = __all_sync(0xffffffffu, arrived);
    if (!arrived && lane == 0) atomicCAS(status, 0, kDevTimeoutCeFused);
  }

  // ---- statistics of this CTA's slice, from shared memory
  CeRowState slice;          // valid in every lane of warp 0 after the block below
  ce_state_init(slice);
  float slice_ref = 0.f;     // kStoreExp: log2(e) * slice maximum, the reference point of the stored exponentials
  auto merge_across_lanes = [](CeRowState& s) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      CeRowState other;
      other.m = __shfl_xor_sync(0xffffffffu, s.m, o);
      other.d = __shfl_xor_sync(0xffffffffu, s.d, o);
      other.ss = __shfl_xor_sync(0xffffffffu, s.ss, o);
      other.best = __shfl_xor_sync(0xffffffffu, s.best, o);
      other.best_idx = __shfl_xor_sync(0xffffffffu, s.best_idx, o);
      ce_state_merge(s, other);
    }
  };
  if constexpr (!kStoreExp) {
    CeRowState st;
    ce_state_init(st);
    if (arrived) {
      for (int i = lane; i < my_vecs; i += 32) {
        const uint4 raw = piece_smem[i];
        const T* e = reinterpret_cast<const T*>(&raw);
        float v[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          v[j] = CeElem<T>::load(e + j);
          if (softcap > 0.f) v[j] = softcap * tanh_accurate(v[j] * inv_softcap);
        }
        ce_state_push_vec<kVec>(st, v, col_weight, (piece_begin + i) * kVec);
      }
    }
    merge_across_lanes(st);
    if (lane == 0) warp_state[warp] = st;
    __syncthreads();
    if (warp == 0) {
      if (lane < kWarps) slice = warp_state[lane];
      merge_across_lanes(slice);
      // the butterfly leaves each lane with the same set merged in its own order: every peer gets lane 0's copy
      slice.m = __shfl_sync(0xffffffffu, slice.m, 0);
      slice.d = __shfl_sync(0xffffffffu, slice.d, 0);
      slice.ss = __shfl_sync(0xffffffffu, slice.ss, 0);
      slice.best = __shfl_sync(0xffffffffu, slice.best, 0);
      slice.best_idx = __shfl_sync(0xffffffffu, slice.best_idx, 0);
    }
  } else {
    // pass 0: maximum and its first position
    float best = -INFINITY;
    int best_idx = 0x7fffffff;
    auto max_across_lanes = [&]() {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
        if (ob > best || (ob == best && oi < best_idx)) {
          best = ob;
          best_idx = oi;
        }
      }
    };
    if (arrived) {
      for (int i = lane; i < my_vecs; i += 32) {
        const uint4 raw = piece_smem[i];
        const T* e = reinterpret_cast<const T*>(&raw);
        float v[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) v[j] = CeElem<T>::load(e + j);
        float vmax = v[0];
#pragma unroll
        for (int j = 1; j < kVec; ++j) vmax = fmaxf(vmax, v[j]);
        if (vmax > best) {   // vectors arrive in increasing order within a lane: strictly greater keeps the lowest index
          int idx = kVec - 1;
#pragma unroll
          for (int j = kVec - 2; j >= 0; --j) idx = (v[j] == vmax) ? j : idx;
          best = vmax;
          best_idx = (piece_begin + i) * kVec + idx;
        }
      }
    }
    max_across_lanes();
    if (lane == 0) {
      warp_max[warp] = best;
      warp_argmax[warp] = best_idx;
    }
    __syncthreads();
    best = lane < kWarps ? warp_max[lane] : -INFINITY;
    best_idx = lane < kWarps ? warp_argmax[lane] : 0x7fffffff;
    max_across_lanes();
    slice_ref = (best == -INFINITY) ? 0.f : best * kLog2e;     // a slice of -inf only: every exponential is 0
    // pass 1: exponentials against the slice maximum, summed in fp32 before they are rounded into the logits' place
    float d = 0.f, ss = 0.f;
    const bool want_sum = rm.alpha > 0.f;       // the (weighted) logit sum only enters the label-smoothing term
    if (arrived) {
      for (int i = lane; i < my_vecs; i += 32) {
        const uint4 raw = piece_smem[i];
        const T* e = reinterpret_cast<const T*>(&raw);
        float v[kVec], ex[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) v[j] = CeElem<T>::load(e + j);
        if (want_sum) {
          const int col0 = (piece_begin + i) * kVec;
#pragma unroll
          for (int j = 0; j < kVec; ++j) ss = col_weight != nullptr ? fmaf(v[j], col_weight[col0 + j], ss) : ss + v[j];
        }
        float part = 0.f;
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          ex[j] = ex2_approx(fmaf(v[j], kLog2e, -slice_ref));
          part += ex[j];
        }
        d += part;
        uint4 packed;
        T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
        for (int j = 0; j < kVec; ++j) CeElem<T>::store(o + j, ex[j]);
        piece_smem[i] = packed;
      }
    }
    // every partial sum is relative to the same slice maximum: plain sums, in a fixed order
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      d += __shfl_xor_sync(0xffffffffu, d, o);
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    if (lane == 0) {
      warp_state[warp].d = d;
      warp_state[warp].ss = ss;
    }
    __syncthreads();
    if (warp == 0) {
      d = lane < kWarps ? warp_state[lane].d : 0.f;
      ss = lane < kWarps ? warp_state[lane].ss : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        d += __shfl_xor_sync(0xffffffffu, d, o);
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
      }
      slice.m = best;
      slice.d = __shfl_sync(0xffffffffu, d, 0);
      slice.ss = __shfl_sync(0xffffffffu, ss, 0);
      slice.best = best;
      slice.best_idx = best_idx;
    }
  }
  if (warp == 0 && lane < static_cast<int>(n_ctas)) {
    // this CTA's five numbers into slot `rank` of every CTA of the cluster (itself included)
    const uint32_t slot = smem_u32(&peer_state[rank]);
    st_shared_cluster_u32(slot + 0, lane, __float_as_uint(slice.m));
    st_shared_cluster_u32(slot + 4, lane, __float_as_uint(slice.d));
    st_shared_cluster_u32(slot + 8, lane, __float_as_uint(slice.ss));
    st_shared_cluster_u32(slot + 12, lane, __float_as_uint(slice.best));
    st_shared_cluster_u32(slot + 16, lane, static_cast<uint32_t>(slice.best_idx));
  }
  cluster_sync();   // arrive has release, wait has acquire semantics: the peers' slots are visible afterwards

  CeRowState rs = peer_state[0];
  for (uint32_t c = 1; c < n_ctas; ++c) ce_state_merge(rs, peer_state[c]);
  const int amax = rs.best_idx == 0x7fffffff ? 0 : rs.best_idx;
  const float lse = rs.m + logf(rs.d);
  if (rank == 0 && threadIdx.x == 0) {
    const size_t n = static_cast<size_t>(n_rows);
    out.rowstats[0 * n + row] = rs.m;
    out.rowstats[1 * n + row] = rs.d;
    out.rowstats[2 * n + row] = xy;
    out.rowstats[3 * n + row] = rs.ss;
    out.rowstats[4 * n + row] = rs.best;
    reinterpret_cast<int*>(out.rowstats)[5 * n + row] = amax;
    finalize_row(row, rm, t, col_weight, rs.m, rs.d, xy, rs.ss, amax, norm_here, out.lse, out.target_prob, out.loss_rows,
                 out.z_rows, out.correct_rows, out.predicted);
  }
  float ca, cb, cc;
  row_coefs(rm, t, col_weight, lse, expf(xy - lse), norm_here, 1.f, ca, cb, cc);

  // ---- the gradient replaces what the piece holds, which then leaves as one bulk store
  if (arrived && my_vecs > 0) {
    const float l2 = lse * kLog2e;
    const float e_scale = ca * ex2_approx(slice_ref - l2);     // kStoreExp: stored exponential -> c1 * softmax
    const float target_grad = fmaf(ex2_approx(fmaf(xy, kLog2e, -l2)), ca, -cc);   // without the smoothing term
    const int t_vec = (t >= 0 && t < n_cols) ? static_cast<int>(t / kVec) : -1;
    for (int i = lane; i < my_vecs; i += 32) {
      const uint4 raw = piece_smem[i];
      const T* e = reinterpret_cast<const T*>(&raw);
      const int col0 = (piece_begin + i) * kVec;
      float g[kVec];
      if constexpr (kStoreExp) {
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          const float wj = col_weight != nullptr ? col_weight[col0 + j] : 1.f;
          g[j] = fmaf(CeElem<T>::load(e + j), e_scale, -cb * wj);
        }
        if (piece_begin + i == t_vec) {
          const int jt = static_cast<int>(t - static_cast<long long>(col0));
          const float wt = col_weight != nullptr ? col_weight[t] : 1.f;
#pragma unroll
          for (int j = 0; j < kVec; ++j)
            if (j == jt) g[j] = fmaf(-cb, wt, target_grad);
        }
      } else {
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          const float z = CeElem<T>::load(e + j);
          float s = z, chain = 1.f;
          if (softcap > 0.f) {
            const float th = tanh_accurate(z * inv_softcap);
            s = softcap * th;
            chain = fmaf(-th, th, 1.f);
          }
          const float wj = col_weight != nullptr ? col_weight[col0 + j] : 1.f;
          float v = fmaf(ex2_approx(fmaf(s, kLog2e, -l2)), ca, -cb * wj);
          if (static_cast<long long>(col0 + j) == t) v -= cc;
          g[j] = v * chain;
        }
      }
      uint4 packed;
      T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
      for (int j = 0; j < kVec; ++j) CeElem<T>::store(o + j, g[j]);
      piece_smem[i] = packed;
    }
    fence_proxy_async_smem();   // this lane's shared-memory writes, for the bulk store lane 0 issues below
    __syncwarp();
    if (lane == 0) {
      bulk_store_1d(reinterpret_cast<uint4*>(grow) + piece_begin, smem_u32(piece_smem), my_bytes);
      bulk_commit_group();
      bulk_wait_group_read<0>();   // the piece must stay allocated until the store has read it; the write itself is
                                   // complete, like every memory operation of the grid, when the grid is
    }
  }
}

// gradient already formed with an upstream gradient of 1: fold the real one in (what the reference's backward does,
// src/liger_kernel/ops/cross_entropy.py:484-502).  A scalar upstream gradient equal to 1 is detected on the device and
// the launch returns at once, so the caller never has to look at the value on the host.
template <typename T>
__global__ void __launch_bounds__(256)
ce_scale_gradient_kernel(T* grad, long long ld, int n_rows, int n_cols, const float* grad_output, int per_row) {
  constexpr int kVec = CeElem<T>::kVec;
  if (!per_row && grad_output[0] == 1.f) return;
  // a fixed, small grid strides over (row, 256-vector segment) items, so the launch that finds nothing to do is cheap
  const int segs = (n_cols + 256 * kVec - 1) / (256 * kVec);
  const long long items = static_cast<long long>(n_rows) * segs;
  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const int row = static_cast<int>(item / segs);
    const int seg = static_cast<int>(item - static_cast<long long>(row) * segs);
    const float go = per_row ? grad_output[row] : grad_output[0];
    T* g = grad + static_cast<size_t>(row) * ld;
    const int col0 = (seg * 256 + threadIdx.x) * kVec;
    if (col0 + kVec <= n_cols && (reinterpret_cast<uintptr_t>(g + col0) & 15u) == 0) {
      float v[kVec];
      ce_load_vec<T>(g + col0, v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) v[j] *= go;
      ce_store_vec<T>(g + col0, v);
    } else {
      for (int j = 0; j < kVec && col0 + j < n_cols; ++j) CeElem<T>::store(g + col0 + j, CeElem<T>::load(g + col0 + j) * go);
    }
  }
}

}  // namespace flce
