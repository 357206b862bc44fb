// Register epilogues plugged into the tcgen05 main loop (gemm_sm100.cuh).  Each epilogue
// thread owns one output row of the tile and sees its 256 fp32 accumulators 32 at a time.
#pragma once

#include "simt_common.cuh"
#ifdef FLCE_HOST_EMULATION
struct CUtensorMap_st;
typedef struct CUtensorMap_st CUtensorMap;   // the host emulation never dereferences one
#else
#include "ptx_sm100.cuh"
#endif

namespace flce {

// 32 fp32 values -> 32 16-bit values (64 bytes) at dst; one format branch for the whole row segment
__device__ __forceinline__ void store32_16bit(uint4* dst, const float (&g)[32], int fmt) {
  if (fmt == kOutBf16) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __nv_bfloat162 h0 = __floats2bfloat162_rn(g[8 * q + 0], g[8 * q + 1]);
      __nv_bfloat162 h1 = __floats2bfloat162_rn(g[8 * q + 2], g[8 * q + 3]);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(g[8 * q + 4], g[8 * q + 5]);
      __nv_bfloat162 h3 = __floats2bfloat162_rn(g[8 * q + 6], g[8 * q + 7]);
      dst[q] = make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                          *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
    }
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __half2 h0 = __floats2half2_rn(g[8 * q + 0], g[8 * q + 1]);
      __half2 h1 = __floats2half2_rn(g[8 * q + 2], g[8 * q + 3]);
      __half2 h2 = __floats2half2_rn(g[8 * q + 4], g[8 * q + 5]);
      __half2 h3 = __floats2half2_rn(g[8 * q + 6], g[8 * q + 7]);
      dst[q] = make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                          *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
    }
  }
}

// Largest exponent (natural log units) the exp-store form of sweep 1 writes: exp(60) times a vocabulary-long sum stays far
// inside fp32, and with the reference point 40 above the target logit a row would need a loss of 100 nats to reach it.
constexpr float kExpStoreClamp = 60.f;
constexpr float kExpStoreOffset = 40.f;
// lse - shift above this (a loss above 90 nats with the offset of 40) sends the chunk through sweep 1 once more with
// shift = lse, where every stored value is a probability
constexpr float kExpStoreRedoLimit = 50.f;

// =====================================================================================
// Sweep 1: logits tile -> per-(row, tile) softmax statistics.  Nothing of size N x V is stored.
// Feature tests are hoisted out of the per-element loops: each optional stage is one uniform
// branch around a fully unrolled, branch-free pass over the 32 values.
// =====================================================================================
struct StatsEpilogue {
  static constexpr bool kDeepPrefetch = false;
  static constexpr bool kSplitK = false;
  struct Params {
    const long long* target;  // [M] global class ids
    const float* bias;        // [n_cols] or null
    const float* col_weight;  // [n_cols] class weights or null (weights the logit sum only)
    float softcap, inv_softcap;
    int n_cols;               // valid columns (vocabulary rows held by this rank)
    long long vocab_offset;   // global id of column 0
    int m_rows;               // M
    float* pmax;              // [n_tiles][M]
    float* psum;              // [n_tiles][M]
    float* plogit_sum;        // [n_tiles][M] or null
    float* pamax_val;         // [n_tiles][M] or null
    int* pamax_idx;           // [n_tiles][M] or null
    float* target_logit;      // [M], written by the one tile that contains the target
    void* logits_out;         // optional [M][ld_logits] 16-bit copy of the soft-capped logits (single-sweep mode) or null
    long long ld_logits;
    int logits_fmt;           // kOutBf16 / kOutFp16
    // With `shift` ([M], a per-row reference point near the row's log-sum-exp) the copy holds, instead of the logits s,
    //   E = exp(min(s - shift, kExpStoreClamp)) * (1 - (s / softcap)^2)      (zeros on rows whose target is ignore_index),
    // i.e. the softmax numerator up to a per-row factor, with the soft-cap chain factor folded in: the gradient GEMMs
    // take it as an operand as it is and the per-row factor exp(shift - lse) moves into their epilogue / other operand.
    // Unlike rounded logits, E keeps a relative accuracy of one 16-bit ulp whatever the logit's magnitude.
    const float* shift;
    long long ignore_index;
  };

  float m, d, ssum, best, shift2;
  int best_idx, row, nt, tgt_local;
  bool row_ok, row_live;

  __device__ __forceinline__ void begin(const Params& p, int row_, int /*col0*/, int n_tile, bool ok) {
    row = row_;
    nt = n_tile;
    row_ok = ok;
    m = -INFINITY;
    d = 0.f;
    ssum = 0.f;
    best = -INFINITY;
    best_idx = 0;
    tgt_local = -1;
    shift2 = 0.f;
    row_live = false;
    if (ok) {
      const long long y = p.target[row];
      const long long t = y - p.vocab_offset;
      if (t >= 0 && t < p.n_cols) tgt_local = static_cast<int>(t);
      if (p.shift != nullptr) {
        shift2 = p.shift[row] * kLog2e;
        row_live = y != p.ignore_index;
      }
    }
  }

  __device__ __forceinline__ void chunk(const Params& p, const uint32_t (&acc)[32], int col, float* /*stage*/, const CUtensorMap* /*map_d*/) {
    float s[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) s[j] = __uint_as_float(acc[j]);
    const bool ragged = col + 32 > p.n_cols;
    if (p.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) s[j] += __ldg(p.bias + min(col + j, p.n_cols - 1));
    }
    if (p.softcap > 0.f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) s[j] = p.softcap * tanh_accurate(s[j] * p.inv_softcap);
    }
    if (p.logits_out != nullptr && p.shift == nullptr && row_ok)
      store32_16bit(reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.logits_out) + static_cast<size_t>(row) * p.ld_logits + col),
                    s, p.logits_fmt);
    if (p.logits_out != nullptr && p.shift != nullptr && row_ok) {
      float e[32];
      if (row_live) {
        const float lim = kExpStoreClamp * kLog2e;
#pragma unroll
        for (int j = 0; j < 32; ++j) e[j] = ex2_approx(fminf(fmaf(s[j], kLog2e, -shift2), lim));
        if (p.softcap > 0.f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float th = s[j] * p.inv_softcap;
            e[j] *= fmaf(-th, th, 1.f);
          }
        }
        if (ragged) {
#pragma unroll
          for (int j = 0; j < 32; ++j) e[j] = (col + j < p.n_cols) ? e[j] : 0.f;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) e[j] = 0.f;
      }
      store32_16bit(reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.logits_out) + static_cast<size_t>(row) * p.ld_logits + col),
                    e, p.logits_fmt);
    }
    if (ragged) {
#pragma unroll
      for (int j = 0; j < 32; ++j) s[j] = (col + j < p.n_cols) ? s[j] : -INFINITY;
    }
    // chunk maximum: four independent chains
    float c0 = fmaxf(s[0], s[4]), c1 = fmaxf(s[1], s[5]), c2 = fmaxf(s[2], s[6]), c3 = fmaxf(s[3], s[7]);
#pragma unroll
    for (int j = 8; j < 32; j += 4) {
      c0 = fmaxf(c0, s[j]);
      c1 = fmaxf(c1, s[j + 1]);
      c2 = fmaxf(c2, s[j + 2]);
      c3 = fmaxf(c3, s[j + 3]);
    }
    const float cm = fmaxf(fmaxf(c0, c1), fmaxf(c2, c3));
    if (p.pamax_val != nullptr && cm > best) {  // strictly greater: ties keep the lowest index
      int idx = 31;
#pragma unroll
      for (int j = 30; j >= 0; --j) idx = (s[j] == cm) ? j : idx;
      best = cm;
      best_idx = static_cast<int>(p.vocab_offset) + col + idx;  // global class id
    }
    if (p.plogit_sum != nullptr) {
      float a0 = 0.f, a1 = 0.f;
      if (p.col_weight != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float w0 = __ldg(p.col_weight + min(col + j, p.n_cols - 1));
          const float w1 = __ldg(p.col_weight + min(col + j + 1, p.n_cols - 1));
          a0 = fmaf((col + j < p.n_cols) ? s[j] : 0.f, w0, a0);
          a1 = fmaf((col + j + 1 < p.n_cols) ? s[j + 1] : 0.f, w1, a1);
        }
      } else if (ragged) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          a0 += (col + j < p.n_cols) ? s[j] : 0.f;
          a1 += (col + j + 1 < p.n_cols) ? s[j + 1] : 0.f;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          a0 += s[j];
          a1 += s[j + 1];
        }
      }
      ssum += a0 + a1;
    }
    const float m_new = fmaxf(m, cm);
    const float ml2 = m_new * kLog2e;
    float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      p0 += ex2_approx(fmaf(s[j], kLog2e, -ml2));
      p1 += ex2_approx(fmaf(s[j + 1], kLog2e, -ml2));
      p2 += ex2_approx(fmaf(s[j + 2], kLog2e, -ml2));
      p3 += ex2_approx(fmaf(s[j + 3], kLog2e, -ml2));
    }
    d = fmaf(d, ex2_approx((m - m_new) * kLog2e), (p0 + p1) + (p2 + p3));
    m = m_new;
    const unsigned rel = static_cast<unsigned>(tgt_local - col);
    if (rel < 32u) {
      float sy = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) sy = (rel == static_cast<unsigned>(j)) ? s[j] : sy;
      p.target_logit[row] = sy;
    }
  }

  __device__ __forceinline__ void end(const Params& p) {
    if (!row_ok) return;
    const size_t o = static_cast<size_t>(nt) * p.m_rows + row;
    p.pmax[o] = m;
    p.psum[o] = d;
    if (p.plogit_sum != nullptr) p.plogit_sum[o] = ssum;
    if (p.pamax_val != nullptr) {
      p.pamax_val[o] = best;
      p.pamax_idx[o] = best_idx;
    }
  }
};

// =====================================================================================
// Sweep 2: recomputed logits tile -> logit gradient dZ (16-bit) in the slab workspace.
//   dZ[r, j] = (p[r, j] * c1[r] - c2[r] * colw[j] - c3[r] * [j == target_r]) * (1 - tanh^2) ,
// with p = exp(s - lse); c1/c2/c3 carry every per-row factor (normalisers, z-loss, smoothing,
// class weight of the target, token scaling, upstream gradient, ignored rows = 0).
// =====================================================================================
struct DzEpilogue {
  static constexpr bool kDeepPrefetch = false;
  static constexpr bool kSplitK = false;
  struct Params {
    const long long* target;
    const float* bias;
    const float* col_weight;
    float softcap, inv_softcap;
    int n_cols;               // valid columns of this slab
    long long vocab_offset;   // global id of slab column 0
    int m_rows;
    const float* lse;         // [M]
    const float* c1;          // [M]
    const float* c2;          // [M]
    const float* c3;          // [M]
    void* dz;                 // [M][ld_dz] 16-bit
    void* dz_lo;              // optional second slab: 16-bit rounding residual of dz (fp32-input path), or null
    long long ld_dz;
    int out_fmt;              // kOutBf16 / kOutFp16
  };

  float l2, c1, c2, c3;
  int row, tgt_local;
  bool row_ok;

  __device__ __forceinline__ void begin(const Params& p, int row_, int /*col0*/, int /*n_tile*/, bool ok) {
    row = row_;
    row_ok = ok;
    tgt_local = -1;
    l2 = 0.f;
    c1 = c2 = c3 = 0.f;
    if (ok) {
      const long long t = p.target[row] - p.vocab_offset;
      if (t >= 0 && t < p.n_cols) tgt_local = static_cast<int>(t);
      l2 = p.lse[row] * kLog2e;
      c1 = p.c1[row];
      c2 = p.c2[row];
      c3 = p.c3[row];
    }
  }

  __device__ __forceinline__ void chunk(const Params& p, const uint32_t (&acc)[32], int col, float* /*stage*/, const CUtensorMap* /*map_d*/) {
    if (!row_ok) return;
    float g[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) g[j] = __uint_as_float(acc[j]);
    if (p.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) g[j] += __ldg(p.bias + min(col + j, p.n_cols - 1));
    }
    const bool capped = p.softcap > 0.f;
    if (capped) {
#pragma unroll
      for (int j = 0; j < 32; ++j) g[j] = p.softcap * tanh_accurate(g[j] * p.inv_softcap);
    }
    // true-class correction, formed in fp32 before rounding: c3, times the soft-cap chain factor at the target
    const unsigned rel = static_cast<unsigned>(tgt_local - col);
    float corr = c3;
    if (rel < 32u && capped) {
      float sy = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) sy = (rel == static_cast<unsigned>(j)) ? g[j] : sy;
      const float thy = sy * p.inv_softcap;
      corr = c3 * fmaf(-thy, thy, 1.f);
    }
    // g holds the soft-capped logits s; turn them into gradients in place
    if (p.col_weight != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float wj = __ldg(p.col_weight + min(col + j, p.n_cols - 1));
        const float s = g[j];
        float v = fmaf(ex2_approx(fmaf(s, kLog2e, -l2)), c1, -c2 * wj);
        if (capped) {
          const float th = s * p.inv_softcap;
          v *= fmaf(-th, th, 1.f);
        }
        g[j] = v;
      }
    } else if (capped) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float s = g[j];
        const float th = s * p.inv_softcap;
        g[j] = fmaf(ex2_approx(fmaf(s, kLog2e, -l2)), c1, -c2) * fmaf(-th, th, 1.f);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) g[j] = fmaf(ex2_approx(fmaf(g[j], kLog2e, -l2)), c1, -c2);
    }
    if (rel < 32u) {
#pragma unroll
      for (int j = 0; j < 32; ++j) g[j] = (rel == static_cast<unsigned>(j)) ? g[j] - corr : g[j];
    }
    if (col + 32 > p.n_cols) {
#pragma unroll
      for (int j = 0; j < 32; ++j) g[j] = (col + j < p.n_cols) ? g[j] : 0.f;
    }
    store32_16bit(reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.dz) + static_cast<size_t>(row) * p.ld_dz + col), g,
                  p.out_fmt);
    if (p.dz_lo != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float hi = (p.out_fmt == kOutBf16) ? __bfloat162float(__float2bfloat16_rn(g[j])) : __half2float(__float2half_rn(g[j]));
        g[j] -= hi;
      }
      store32_16bit(reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.dz_lo) + static_cast<size_t>(row) * p.ld_dz + col), g,
                    p.out_fmt);
    }
  }

  __device__ __forceinline__ void end(const Params&) {}
};

// =====================================================================================
// Scaled cross-entropy (negative log-likelihood + entropy of softmax(z / T)) on the same two sweeps.
// Sweep 1 keeps, per (row, tile), max, sum exp(s - max) and sum exp(s - max) * s with s = z * scale; the entropy is
// lse - (sum e s) / (sum e).  Sweep 2 turns the recomputed logits into
//   dZ[r, j] = (p[r, j] * (a_r + b_r * s[r, j]) - c_r * [j == target_r]),   p = exp(s - lse_r),
//   a = (g_nll - g_ent * (H - lse)) * scale,  b = -g_ent * scale,  c = g_nll * scale     (zero on ignored rows),
// which is d(nll * g_nll + entropy * g_ent) / dz.
// =====================================================================================
struct EntropyStatsEpilogue {
  static constexpr bool kDeepPrefetch = false;
  static constexpr bool kSplitK = false;
  struct Params {
    const long long* target;  // [M] class ids
    float scale;              // 1 / temperature
    int n_cols;               // valid columns
    int m_rows;               // M
    float* pmax;              // [n_tiles][M]
    float* psum;              // [n_tiles][M]
    float* pts;               // [n_tiles][M]  sum exp(s - max) * s
    float* target_logit;      // [M] scaled logit of the target, written by the one tile that contains it
  };

  float m, d, t;
  int row, nt, tgt_local;
  bool row_ok;

  __device__ __forceinline__ void begin(const Params& p, int row_, int /*col0*/, int n_tile, bool ok) {
    row = row_;
    nt = n_tile;
    row_ok = ok;
    m = -INFINITY;
    d = 0.f;
    t = 0.f;
    tgt_local = -1;
    if (ok) {
      const long long y = p.target[row];
      if (y >= 0 && y < p.n_cols) tgt_local = static_cast<int>(y);
    }
  }

  __device__ __forceinline__ void chunk(const Params& p, const uint32_t (&acc)[32], int col, float* /*stage*/, const CUtensorMap* /*map_d*/) {
    float s[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) s[j] = __uint_as_float(acc[j]) * p.scale;
    const bool ragged = col + 32 > p.n_cols;
    float c0 = -INFINITY, c1 = -INFINITY, c2 = -INFINITY, c3 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      c0 = fmaxf(c0, (!ragged || col + j < p.n_cols) ? s[j] : -INFINITY);
      c1 = fmaxf(c1, (!ragged || col + j + 1 < p.n_cols) ? s[j + 1] : -INFINITY);
      c2 = fmaxf(c2, (!ragged || col + j + 2 < p.n_cols) ? s[j + 2] : -INFINITY);
      c3 = fmaxf(c3, (!ragged || col + j + 3 < p.n_cols) ? s[j + 3] : -INFINITY);
    }
    const float m_new = fmaxf(m, fmaxf(fmaxf(c0, c1), fmaxf(c2, c3)));
    const float ml2 = m_new * kLog2e;
    float p0 = 0.f, p1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const bool v0 = !ragged || col + j < p.n_cols, v1 = !ragged || col + j + 1 < p.n_cols;
      const float e0 = v0 ? ex2_approx(fmaf(s[j], kLog2e, -ml2)) : 0.f;
      const float e1 = v1 ? ex2_approx(fmaf(s[j + 1], kLog2e, -ml2)) : 0.f;
      p0 += e0;
      p1 += e1;
      q0 = fmaf(e0, v0 ? s[j] : 0.f, q0);
      q1 = fmaf(e1, v1 ? s[j + 1] : 0.f, q1);
    }
    const float keep = ex2_approx((m - m_new) * kLog2e);
    d = fmaf(d, keep, p0 + p1);
    t = fmaf(t, keep, q0 + q1);
    m = m_new;
    const unsigned rel = static_cast<unsigned>(tgt_local - col);
    if (rel < 32u) {
      float sy = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) sy = (rel == static_cast<unsigned>(j)) ? s[j] : sy;
      p.target_logit[row] = sy;
    }
  }

  __device__ __forceinline__ void end(const Params& p) {
    if (!row_ok) return;
    const size_t o = static_cast<size_t>(nt) * p.m_rows + row;
    p.pmax[o] = m;
    p.psum[o] = d;
    p.pts[o] = t;
  }
};

struct ScaledDzEpilogue {
  static constexpr bool kDeepPrefetch = false;
  static constexpr bool kSplitK = false;
  struct Params {
    const long long* target;
    long long ignore_index;
    float scale;              // 1 / temperature
    int n_cols;               // valid columns of this slab
    long long vocab_offset;   // class id of slab column 0
    int m_rows;
    const float* lse;         // [M]
    const float* entropy;     // [M]
    const float* grad_nll;    // [M] or null
    const float* grad_entropy;  // [M] or null
    void* dz;                 // [M][ld_dz] 16-bit
    long long ld_dz;
    int out_fmt;
  };

  float l2, a, b, c;
  int row, tgt_local;
  bool row_ok;

  __device__ __forceinline__ void begin(const Params& p, int row_, int /*col0*/, int /*n_tile*/, bool ok) {
    row = row_;
    row_ok = ok;
    tgt_local = -1;
    l2 = 0.f;
    a = b = c = 0.f;
    if (ok) {
      const long long y = p.target[row];
      const float lse = p.lse[row];
      l2 = lse * kLog2e;
      if (y != p.ignore_index) {
        const long long local = y - p.vocab_offset;
        if (local >= 0 && local < p.n_cols) tgt_local = static_cast<int>(local);
        const float gn = p.grad_nll != nullptr ? p.grad_nll[row] : 0.f;
        const float ge = p.grad_entropy != nullptr ? p.grad_entropy[row] : 0.f;
        a = (gn - ge * (p.entropy[row] - lse)) * p.scale;
        b = -ge * p.scale;
        c = gn * p.scale;
      }
    }
  }

  __device__ __forceinline__ void chunk(const Params& p, const uint32_t (&acc)[32], int col, float* /*stage*/, const CUtensorMap* /*map_d*/) {
    if (!row_ok) return;
    float g[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float s = __uint_as_float(acc[j]) * p.scale;
      g[j] = ex2_approx(fmaf(s, kLog2e, -l2)) * fmaf(b, s, a);
    }
    const unsigned rel = static_cast<unsigned>(tgt_local - col);
    if (rel < 32u) {
#pragma unroll
      for (int j = 0; j < 32; ++j) g[j] = (rel == static_cast<unsigned>(j)) ? g[j] - c : g[j];
    }
    if (col + 32 > p.n_cols) {
#pragma unroll
      for (int j = 0; j < 32; ++j) g[j] = (col + j < p.n_cols) ? g[j] : 0.f;
    }
    store32_16bit(reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.dz) + static_cast<size_t>(row) * p.ld_dz + col), g,
                  p.out_fmt);
  }

  __device__ __forceinline__ void end(const Params&) {}
};

// =====================================================================================
// Plain store / accumulate epilogue for the two gradient GEMMs.
//   acc_in  != null : v += acc_in[row][col]     (fp32 partial from earlier slabs)
//   acc_out != null : acc_out[row][col] = v     (fp32 partial for later slabs)
//   out     != null : out[row][col] = cast(v)   (final result, out_fmt)
// n_cols must be a multiple of 8 and ld_* keep rows 16-byte aligned.
// Optional, applied to the accumulator before anything else (the exp-store form of the single-sweep mode):
//   row_scale != null : v *= row_scale[row]                       (per-row softmax factor of grad_input)
//   r1_col    != null : v -= r1_row[row] * r1_col[col]            (r1_row null = 1; the uniform label-smoothing term,
//                                                                  a rank-1 matrix, never formed)
// =====================================================================================
struct StoreEpilogue {
  static constexpr bool kDeepPrefetch = true;
  // a tile's K range may be cut in two, the second part added to what the first one wrote (fp32 accumulator output only)
  static constexpr bool kSplitK = true;
  template <class P>
  __device__ static P accumulating(P p) {
    p.acc_add = 1;
    return p;
  }
  struct Params {
    int m_rows, n_cols;
    const float* acc_in;
    float* acc_out;
    long long ld_acc;
    void* out;
    long long ld_out;
    int out_fmt;
    const float* row_scale;
    const float* r1_row;
    const float* r1_col;
    // 1: add into acc_out with vector reductions at L2 (no read in this kernel, nothing to wait for); acc_in must be null.
    // Every element is owned by one thread of one launch, so the sum over launches keeps the stream's order.
    int acc_add;
    // 1 (set by the launcher when exactly one of out / acc_out is written and nothing is read back): each 32 x 32 patch
    // leaves through a TMA store (or TMA add, with acc_add) from the warp's shared-memory stage, described by the
    // kernel's output tensor map; the warp only writes shared memory and issues one bulk copy per patch.
    int bulk;
  };

  int row, flip;
  bool row_ok;
  float scale, r1;

  __device__ __forceinline__ void begin(const Params& p, int row_, int, int, bool ok) {
    row = row_;
    row_ok = ok;
    flip = 0;
#ifndef FLCE_HOST_EMULATION
    if (p.bulk) {   // both stage buffers are free again before this tile's first patch (tiles may end on either one)
      if ((threadIdx.x & 31) == 0) bulk_wait_group_read<0>();
      __syncwarp();
    }
#endif
    scale = 1.f;
    r1 = 0.f;
    if (ok) {
      if (p.row_scale != nullptr) scale = p.row_scale[row];
      if (p.r1_col != nullptr) r1 = p.r1_row != nullptr ? p.r1_row[row] : 1.f;
    }
  }

  // The accumulators arrive one output row per thread.  Written out like that, every load / store instruction of the
  // warp touches 32 different rows, 16 bytes each; with an fp32 partial to read and to write per element that costs
  // more than the main loop of a short-K tile saves.  So the 32 x 32 patch goes through the warp's shared-memory
  // stage: afterwards 8 lanes cover 32 consecutive columns of one row, 4 rows per instruction, and every global access
  // is a whole 128-byte (fp32) or 64-byte (16-bit) row segment.
  __device__ __forceinline__ void chunk(const Params& p, const uint32_t (&acc)[32], int col, float* stage,
                                        const CUtensorMap* map_d) {
    const int lane = threadIdx.x & 31;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
    if (p.row_scale != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= scale;
    }
    if (p.r1_col != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = fmaf(-r1, __ldg(p.r1_col + min(col + j, p.n_cols - 1)), v[j]);
    }
    if (p.bulk) {
      void* dst_base = p.acc_out != nullptr ? static_cast<void*>(p.acc_out) : p.out;
      const long long ld = p.acc_out != nullptr ? p.ld_acc : p.ld_out;
      const int fmt = p.acc_out != nullptr ? static_cast<int>(kOutFp32) : p.out_fmt;
#ifdef FLCE_HOST_EMULATION
      // what the bulk copy does, element by element: the patch clipped to the output's extents, stored or added
      (void)stage;
      (void)map_d;
      if (row < p.m_rows) {
        for (int j = 0; j < 32 && col + j < p.n_cols; ++j) {
          const size_t at = static_cast<size_t>(row) * ld + col + j;
          if (fmt == kOutFp32) {
            float* d = static_cast<float*>(dst_base) + at;
            *d = p.acc_add ? *d + v[j] : v[j];
          } else {
            static_cast<uint16_t*>(dst_base)[at] = static_cast<uint16_t>(pack2(v[j], 0.f, fmt) & 0xffffu);
          }
        }
      }
#else
      (void)dst_base;
      (void)ld;
      uint8_t* buf = reinterpret_cast<uint8_t*>(stage) + (flip ? 4096 : 0);
      flip ^= 1;
      if (lane == 0) bulk_wait_group_read<1>();   // the copy that last read this buffer (two patches ago) is done with it
      __syncwarp();
      if (fmt == kOutFp32) {
        // 128-byte rows under the 128-byte swizzle of the tensor map: 16-byte chunk q of row r sits at position q ^ (r & 7)
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(buf + lane * 128 + ((q ^ (lane & 7)) << 4)) =
              make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      } else {
        store32_16bit(reinterpret_cast<uint4*>(buf + lane * 64), v, fmt);   // dense 64-byte rows, no swizzle
      }
      fence_proxy_async_smem();
      __syncwarp();
      const int row0 = row - lane;
      if (lane == 0 && row0 < p.m_rows) {
        if (p.acc_add) tma_reduce_add_2d(map_d, smem_u32(buf), col, row0);
        else tma_store_2d(map_d, smem_u32(buf), col, row0);
        bulk_commit_group();
      }
#endif
      return;
    }
    float4* mine = reinterpret_cast<float4*>(stage + lane * 36);
#pragma unroll
    for (int q = 0; q < 8; ++q) mine[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    __syncwarp();
    const int row0 = row - lane;                 // first row of this warp's patch
    const int c4 = (lane & 7) * 4;               // this lane's four columns inside the patch
    const bool col_ok = col + c4 < p.n_cols;     // n_cols is a multiple of 8: a group of four is in or out as a whole
    const int r_first = lane >> 3;
    // partial-sum loads four at a time (independent, in flight together), then the arithmetic and the stores: left in
    // program order they would each wait for the store before them (acc_in and acc_out may be the same buffer)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float4 part[4];
      if (p.acc_in != nullptr) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int grow = row0 + (half * 4 + i) * 4 + r_first;
          part[i] = (grow < p.m_rows && col_ok)
                        ? *reinterpret_cast<const float4*>(p.acc_in + static_cast<size_t>(grow) * p.ld_acc + col + c4)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = (half * 4 + i) * 4 + r_first;
        const int grow = row0 + r;
        if (grow < p.m_rows && col_ok) {
          float4 a = *reinterpret_cast<const float4*>(stage + r * 36 + c4);
          if (p.acc_in != nullptr) {
            a.x += part[i].x;
            a.y += part[i].y;
            a.z += part[i].z;
            a.w += part[i].w;
          }
          if (p.acc_out != nullptr) {
            float4* dst = reinterpret_cast<float4*>(p.acc_out + static_cast<size_t>(grow) * p.ld_acc + col + c4);
            if (p.acc_add) vector_add_f32x4(dst, a);
            else *dst = a;
          }
          if (p.out != nullptr) {
            if (p.out_fmt == kOutFp32) {
              *reinterpret_cast<float4*>(static_cast<float*>(p.out) + static_cast<size_t>(grow) * p.ld_out + col + c4) = a;
            } else {
              uint2 o;
              o.x = pack2(a.x, a.y, p.out_fmt);
              o.y = pack2(a.z, a.w, p.out_fmt);
              *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.out) + static_cast<size_t>(grow) * p.ld_out + col + c4) = o;
            }
          }
        }
      }
    }
    __syncwarp();                                // the stage is rewritten by the next chunk
  }

  __device__ __forceinline__ void end(const Params&) {}
};

}  // namespace flce
