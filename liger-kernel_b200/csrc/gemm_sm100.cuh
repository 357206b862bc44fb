// Persistent, warp-specialised tcgen05 GEMM main loop with a pluggable register epilogue.
//
//   D[m, n] = sum_k A[m, k] * B[n, k]          (fp16/bf16 in, fp32 accumulate in tensor memory)
//
// * one CTA (kCtas = 1) or a pair of CTAs on neighbouring SMs (kCtas = 2) owns a
//   (128 * kCtas) x 256 output tile; every CTA keeps its own 128 rows in its own tensor memory;
// * warp 0 streams 64-wide K slices of A and B into a ring of shared-memory stages with TMA
//   (each CTA of a pair loads only its own rows of A and its own half of B: no multicast);
// * warp 1 (of the pair's leader) issues tcgen05.mma and hands stages back through
//   tcgen05.commit -> mbarrier;
// * warps 2..5 drain finished accumulators with tcgen05.ld, 32 columns at a time, one output row
//   per thread, and feed them to the epilogue functor.  Two accumulators (2 x 256 columns)
//   let the epilogue of tile i overlap the main loop of tile i+1.
// * kNSub = 2 (CTA pairs only) widens the tile to 256 x 512: both 256-column accumulators belong to one tile and
//   every K slice of A feeds two MMAs.  A pair then pulls (256 + 512) x 64 elements from L2 per 256 x 512 x 64
//   products instead of (256 + 256) x 64 per 256 x 256 x 64: 48 instead of 64 bytes per clock and SM at full tensor
//   rate, under what the L2 -> SM path delivers without cluster multicast.  The epilogue no longer overlaps the next
//   tile's main loop, so this form is for long K and light epilogues (the two gradient GEMMs).
//
// Either operand may be K-major (K contiguous in global memory) or MN-major (M or N
// contiguous); the latter is what the weight-gradient GEMM (dZ^T X) and the B side of the
// input-gradient GEMM (dZ W) need, so no transposed copies are ever made.
//
// Ragged edges are handled by TMA zero fill on loads (the tensor maps carry the exact extents)
// and by bounds checks in the epilogues.
#pragma once

#include "ptx_sm100.cuh"
#include "tile_schedule.cuh"

namespace flce {

enum Major : int { kMajorK = 0, kMajorMN = 1 };

// Optional cycle accounting for tuning (compile with -DFLCE_CLOCK_TRACE): per CTA, cycles the three roles
// spend waiting on each barrier and cycles the epilogue is busy.  Off in the shipped library.
#ifdef FLCE_CLOCK_TRACE
__device__ unsigned long long g_clock_trace[1024 * 8];
#define FLCE_TRACE_DECL(name) long long name = 0
#define FLCE_TRACE_BEGIN(t) const long long t = clock64()
#define FLCE_TRACE_ADD(acc, t) acc += clock64() - t
#define FLCE_TRACE_STORE(slot, v) g_clock_trace[(blockIdx.x & 1023) * 8 + slot] = static_cast<unsigned long long>(v)
#else
#define FLCE_TRACE_DECL(name)
#define FLCE_TRACE_BEGIN(t)
#define FLCE_TRACE_ADD(acc, t)
#define FLCE_TRACE_STORE(slot, v)
#endif

constexpr int kUmmaK = 16;
constexpr int kNumThreads = 192;  // 6 warps
constexpr int kNumEpilogueWarps = 4;
constexpr int kTmemCols = 512;    // two 256-column accumulators

template <int kCtas, int kNSub = 1>
struct StageCfg {
  static_assert(kNSub == 1 || (kNSub == 2 && kCtas == 2), "the 512-column tile exists for CTA pairs only");
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBRows = kNSub * kBlockN / kCtas;             // rows of B this CTA stages per K slice
  static constexpr int kBBytes = kBRows * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (kNSub == 2) ? 4 : ((kCtas == 1) ? 4 : 6);
  static constexpr int kAccStages = (kNSub == 2) ? 1 : 2;            // accumulators in flight (tensor memory: 512 columns)
  static constexpr int kRingBytes = kStages * kStageBytes;
  // per epilogue warp, 8 KiB right behind the ring (so 1 KiB-aligned): two dense 32 x 32 fp32 patches that leave as TMA
  // stores, or one 32 x 36-float patch for the epilogue form that reads partial sums back
  static constexpr int kEpiStageFloats = 2048;
  static constexpr int kEpiStageBytes = kNumEpilogueWarps * kEpiStageFloats * 4;
  // ring + epilogue staging + barriers / bookkeeping, plus 1 KiB so the ring can be aligned to the swizzle atom
  static constexpr int kSmemBytes = kRingBytes + kEpiStageBytes + 256 + 1024;
};

// Epilogue concept:
//   struct Epi {
//     struct Params {...};                                  // trivially copyable, passed by value
//     __device__ void begin(const Params&, int row, int col0, int n_tile, bool row_ok);
//     static constexpr bool kDeepPrefetch;                  // keep two tensor-memory loads in flight (light epilogues)
//     __device__ void chunk(const Params&, const uint32_t (&acc)[32], int col, float* stage, const CUtensorMap* map_d);
//                         // fp32 bit patterns; stage: this warp's 8 KiB of shared memory; map_d: tensor map of the output
//                         // (valid when the launcher set Params::bulk); called by all 32 lanes together
//     __device__ void end(const Params&);
//   };
template <int kCtas, int kAMajor, int kBMajor, class Epi, int kNSub = 1>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_d, const GemmShape shape_arg, const int ab_format,
                    const typename Epi::Params ep, int* status) {
  using Cfg = StageCfg<kCtas, kNSub>;
  constexpr int kTileN = kBlockN * kNSub;          // output columns per tile
  constexpr int kAccStages = Cfg::kAccStages;
  GemmShape shape = shape_arg;
  if (shape.gate != nullptr && *shape.gate == 0) return;   // uniform across the grid; nothing has been set up yet
  if (shape.active_rows != nullptr) limit_to_active_rows(shape, *shape.active_rows - shape.active_base, kCtas);   // uniform across the grid
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  // the swizzle pattern is a function of the address: align the ring to 1024 B
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring_a = smem;
  uint8_t* ring_b = smem + kStages * Cfg::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kRingBytes + Cfg::kEpiStageBytes);
  uint64_t* full_bar = bars;                    // [kStages]  TMA bytes landed
  uint64_t* empty_bar = bars + kStages;         // [kStages]  MMAs that read the stage retired
  uint64_t* tmem_full_bar = bars + 2 * kStages; // [2]        accumulator complete
  uint64_t* tmem_empty_bar = tmem_full_bar + 2; // [2]        accumulator drained
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  float* epi_stage = reinterpret_cast<float*>(smem + Cfg::kRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCtas == 1) ? 0u : cluster_ctarank();
  const bool is_leader = (cta_rank == 0);
  const int unit = blockIdx.x / kCtas;          // tile-owning unit (CTA or CTA pair)
  const int num_units = gridDim.x / kCtas;
  const int num_tiles = shape.m_tiles * shape.n_tiles;
  // the first tile of this unit as two parts [0, split_kb) and [split_kb, k_blocks), the second added to the first's output
  int split_kb = 0;
  if constexpr (kNSub == 2 && Epi::kSplitK) split_kb = stagger_split(shape, unit, num_units);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), kNumEpilogueWarps * kCtas);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc<kCtas>(smem_u32(tmem_base_slot), kTmemCols);
    tmem_relinquish<kCtas>();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_descriptor(&map_a);
    tma_prefetch_descriptor(&map_b);
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCtas == 2) cluster_sync();   // partner's barriers are initialised before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t policy_a = make_l2_policy(shape.hint_a);
      const uint64_t policy_b = make_l2_policy(shape.hint_b);
      FLCE_TRACE_DECL(wait_empty);
      FLCE_TRACE_BEGIN(t_kernel);
      for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
        int mt, nt;
        decode_tile(shape, tile, mt, nt);
        const int m0 = (mt * kCtas + static_cast<int>(cta_rank)) * kBlockM;
        // this CTA's share of sub-tile j of B: rows n0 + j * 256 + [0, 256 / kCtas)
        const int n0 = nt * kTileN + static_cast<int>(cta_rank) * (kBlockN / kCtas);
        for (int kb = 0; kb < shape.k_blocks; ++kb) {
          FLCE_TRACE_BEGIN(t_w);
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, status, kDevTimeoutEmptyBarrier);
          FLCE_TRACE_ADD(wait_empty, t_w);
          if (!ok) break;
          const uint32_t local_full = smem_u32(&full_bar[stage]);
          if (is_leader) mbar_arrive_expect_tx(local_full, Cfg::kStageBytes * kCtas);
          uint32_t signal_bar = local_full;
          if constexpr (kCtas == 2) {
            asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(signal_bar) : "r"(local_full));
          }
          const int k0 = kb * kBlockK;
          const uint32_t dst_a = smem_u32(ring_a + stage * Cfg::kABytes);
          const uint32_t dst_b = smem_u32(ring_b + stage * Cfg::kBBytes);
          auto load = [&](uint32_t dst, const CUtensorMap* map, int x, int y) {
            const bool is_a = (map == &map_a);
            const int hint = is_a ? shape.hint_a : shape.hint_b;
            if (hint == 0) {
              if constexpr (kCtas == 1) tma_load_2d(dst, map, signal_bar, x, y);
              else tma_load_2d_pair(dst, map, signal_bar, x, y);
            } else {
              const uint64_t pol = is_a ? policy_a : policy_b;
              if constexpr (kCtas == 1) tma_load_2d_hint(dst, map, signal_bar, x, y, pol);
              else tma_load_2d_pair_hint(dst, map, signal_bar, x, y, pol);
            }
          };
          if constexpr (kAMajor == kMajorK) {
            load(dst_a, &map_a, k0, m0);                          // box: 64 k x 128 rows
          } else {
#pragma unroll
            for (int i = 0; i < kBlockM / 64; ++i)                 // boxes: 64 m x 64 k
              load(dst_a + i * (64 * kBlockK * 2), &map_a, m0 + i * 64, k0);
          }
          constexpr int kSubRows = kBlockN / kCtas;               // rows of one sub-tile held by this CTA
#pragma unroll
          for (int j = 0; j < kNSub; ++j) {
            const uint32_t dst_bj = dst_b + j * (kSubRows * kBlockK * 2);
            if constexpr (kBMajor == kMajorK) {
              load(dst_bj, &map_b, k0, n0 + j * kBlockN);         // box: 64 k x (256 / kCtas) rows
            } else {
#pragma unroll
              for (int i = 0; i < kSubRows / 64; ++i)              // boxes: 64 n x 64 k
                load(dst_bj + i * (64 * kBlockK * 2), &map_b, n0 + j * kBlockN + i * 64, k0);
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      FLCE_TRACE_STORE(4, wait_empty);
      FLCE_TRACE_DECL(total);
      FLCE_TRACE_ADD(total, t_kernel);
      FLCE_TRACE_STORE(5, total);
      if (!ok) {
        // unwinding: give copies already in flight a bounded chance to land before the CTA exits
        for (int s = 0; s < kStages; ++s)
          for (int spin = 0; spin < (1 << 16) && !mbar_try_wait(smem_u32(&full_bar[s]), 0) &&
                             !mbar_try_wait(smem_u32(&full_bar[s]), 1); ++spin) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && is_leader) {
      const uint32_t idesc = make_idesc_f16(ab_format, kAMajor, kBMajor, kBlockM * kCtas, kBlockN);
      // per-operand descriptor geometry
      constexpr uint32_t kLboA = (kAMajor == kMajorK) ? 16u : 64u * kBlockK * 2u;
      constexpr uint32_t kLboB = (kBMajor == kMajorK) ? 16u : 64u * kBlockK * 2u;
      constexpr uint32_t kSbo = 1024u;
      // start-address advance (in 16-byte units) per 16-deep MMA step
      constexpr uint32_t kStepA = (kAMajor == kMajorK) ? (kUmmaK * 2) / 16 : (kUmmaK * 128) / 16;
      constexpr uint32_t kStepB = (kBMajor == kMajorK) ? (kUmmaK * 2) / 16 : (kUmmaK * 128) / 16;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local_tile = 0;
      bool ok = true;
      FLCE_TRACE_DECL(wait_full);
      FLCE_TRACE_DECL(wait_tmem_empty);
      for (int tile = unit; tile < num_tiles && ok; tile += num_units, ++local_tile) {
        const int acc = (kAccStages == 2) ? (local_tile & 1) : 0;
        const int parts = (local_tile == 0 && split_kb > 0) ? 2 : 1;    // split_kb > 0 only with a single accumulator
        for (int part = 0; part < parts && ok; ++part) {
        const int kb_begin = part == 0 ? 0 : split_kb;
        const int kb_end = (parts == 2 && part == 0) ? split_kb : shape.k_blocks;
        FLCE_TRACE_BEGIN(t_e);
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase[acc] ^ 1u, abort_flag, status, kDevTimeoutTmemEmpty);
        FLCE_TRACE_ADD(wait_tmem_empty, t_e);
        if (!ok) break;
        acc_phase[acc] ^= 1u;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kBlockN);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          FLCE_TRACE_BEGIN(t_f);
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, status, kDevTimeoutFullBarrier);
          FLCE_TRACE_ADD(wait_full, t_f);
          if (!ok) break;
          tcgen05_fence_after();
          const uint64_t desc_a = make_smem_desc(smem_u32(ring_a + stage * Cfg::kABytes), kLboA, kSbo);
          const uint64_t desc_b = make_smem_desc(smem_u32(ring_b + stage * Cfg::kBBytes), kLboB, kSbo);
          constexpr uint32_t kSubStepB = ((kBlockN / kCtas) * kBlockK * 2) / 16;   // next sub-tile of B, in 16-byte units
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
#pragma unroll
            for (int j = 0; j < kNSub; ++j)
              umma_f16<kCtas>(tmem_d + static_cast<uint32_t>(j * kBlockN), desc_a + static_cast<uint64_t>(k * kStepA),
                              desc_b + static_cast<uint64_t>(k * kStepB + j * kSubStepB), idesc,
                              (kb != kb_begin || k != 0) ? 1u : 0u);
          }
          if constexpr (kCtas == 1) umma_commit(smem_u32(&empty_bar[stage]));
          else umma_commit_pair(smem_u32(&empty_bar[stage]), 0x3);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (shape.k_blocks == 0) {
          // no MMA was issued for this tile (no active rows): release the epilogue warps with plain arrivals rather
          // than a commit that has nothing to track
          if constexpr (kCtas == 1) {
            mbar_arrive(smem_u32(&tmem_full_bar[acc]));
          } else {
            mbar_arrive_cluster(smem_u32(&tmem_full_bar[acc]), 0);
            mbar_arrive_cluster(smem_u32(&tmem_full_bar[acc]), 1);
          }
        } else if constexpr (kCtas == 1) {
          umma_commit(smem_u32(&tmem_full_bar[acc]));
        } else {
          umma_commit_pair(smem_u32(&tmem_full_bar[acc]), 0x3);
        }
        }  // part
      }
      FLCE_TRACE_STORE(0, wait_full);
      FLCE_TRACE_STORE(1, wait_tmem_empty);
      FLCE_TRACE_STORE(6, local_tile);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;                         // tensor-memory lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    float* stage = epi_stage + quarter * Cfg::kEpiStageFloats;
    uint32_t acc_phase[2] = {0, 0};
    int local_tile = 0;
    bool ok = true;
    FLCE_TRACE_DECL(wait_tmem_full);
    FLCE_TRACE_DECL(busy);
    for (int tile = unit; tile < num_tiles && ok; tile += num_units, ++local_tile) {
      int mt, nt;
      decode_tile(shape, tile, mt, nt);
      const int acc = (kAccStages == 2) ? (local_tile & 1) : 0;
      const int row = (mt * kCtas + static_cast<int>(cta_rank)) * kBlockM + row_in_tile;
      const int col0 = nt * kTileN;
      const int parts = (local_tile == 0 && split_kb > 0) ? 2 : 1;
      for (int part = 0; part < parts && ok; ++part) {
      typename Epi::Params ep_part = ep;
      if constexpr (Epi::kSplitK) {
        if (part == 1) {
          // what part 0 stored must have landed before anything is added to it
          if (lane == 0) bulk_wait_group_all();
          __syncwarp();
          ep_part = Epi::accumulating(ep);
        }
      }
      FLCE_TRACE_BEGIN(t_w);
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase[acc], abort_flag, status, kDevTimeoutTmemFull,
                     static_cast<uint32_t>(shape.poll_sleep_ns));
      FLCE_TRACE_ADD(wait_tmem_full, t_w);
      if (!ok) break;
      FLCE_TRACE_BEGIN(t_b);
      acc_phase[acc] ^= 1u;
      tcgen05_fence_after();
      Epi epi;
      epi.begin(ep_part, row, col0, nt, row < shape.M);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * kBlockN);
      const int n_chunks = min(kTileN / 32, (shape.N - col0 + 31) / 32);   // uniform across the CTA
      if constexpr (Epi::kDeepPrefetch) {
        // light epilogues are bound by the latency of the tensor-memory loads: two 32-column loads are in flight while
        // two are consumed (four register buffers)
        uint32_t a0[32], a1[32], b0[32], b1[32];
        tmem_ld_32x32(taddr, a0);
        if (1 < n_chunks) tmem_ld_32x32(taddr + 32u, a1);
#pragma unroll 1
        for (int c = 0; c < n_chunks; c += 4) {
          tmem_ld_wait();
          tmem_ld_fence(a0);
          tmem_ld_fence(a1);
          if (c + 2 < n_chunks) tmem_ld_32x32(taddr + static_cast<uint32_t>((c + 2) * 32), b0);
          if (c + 3 < n_chunks) tmem_ld_32x32(taddr + static_cast<uint32_t>((c + 3) * 32), b1);
          if (shape.k_blocks == 0) {   // nothing was accumulated (no active rows): the product is zero
#pragma unroll
            for (int j = 0; j < 32; ++j) a0[j] = a1[j] = 0u;
          }
          epi.chunk(ep_part, a0, col0 + c * 32, stage, &map_d);
          if (c + 1 < n_chunks) epi.chunk(ep_part, a1, col0 + (c + 1) * 32, stage, &map_d);
          if (c + 2 < n_chunks) {
            tmem_ld_wait();
            tmem_ld_fence(b0);
            tmem_ld_fence(b1);
            if (c + 4 < n_chunks) tmem_ld_32x32(taddr + static_cast<uint32_t>((c + 4) * 32), a0);
            if (c + 5 < n_chunks) tmem_ld_32x32(taddr + static_cast<uint32_t>((c + 5) * 32), a1);
            if (shape.k_blocks == 0) {
#pragma unroll
              for (int j = 0; j < 32; ++j) b0[j] = b1[j] = 0u;
            }
            epi.chunk(ep_part, b0, col0 + (c + 2) * 32, stage, &map_d);
            if (c + 3 < n_chunks) epi.chunk(ep_part, b1, col0 + (c + 3) * 32, stage, &map_d);
          }
        }
      } else {
      // two register buffers: the load of the next 32 columns is in flight while the current ones are consumed
      uint32_t va[32], vb[32];
      tmem_ld_32x32(taddr, va);
#pragma unroll 1
      for (int c = 0; c < n_chunks; c += 2) {
        tmem_ld_wait();
        tmem_ld_fence(va);
        if (c + 1 < n_chunks) tmem_ld_32x32(taddr + static_cast<uint32_t>((c + 1) * 32), vb);
        if (shape.k_blocks == 0) {   // nothing was accumulated (no active rows): the product is zero
#pragma unroll
          for (int j = 0; j < 32; ++j) va[j] = 0u;
        }
        epi.chunk(ep_part, va, col0 + c * 32, stage, &map_d);
        if (c + 1 < n_chunks) {
          tmem_ld_wait();
          tmem_ld_fence(vb);
          if (c + 2 < n_chunks) tmem_ld_32x32(taddr + static_cast<uint32_t>((c + 2) * 32), va);
          if (shape.k_blocks == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) vb[j] = 0u;
          }
          epi.chunk(ep_part, vb, col0 + (c + 1) * 32, stage, &map_d);
        }
      }
      }
      epi.end(ep_part);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCtas == 1) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        else mbar_arrive_cluster(smem_u32(&tmem_empty_bar[acc]), 0);
      }
      FLCE_TRACE_ADD(busy, t_b);
      }  // part
    }
    if constexpr (Epi::kDeepPrefetch) {
      if (lane == 0) bulk_wait_group_all();   // this warp's TMA stores have left shared memory and landed
    }
    if (threadIdx.x == 64) {
      FLCE_TRACE_STORE(2, wait_tmem_full);
      FLCE_TRACE_STORE(3, busy);
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();  // the single-lane role loops above diverged; the cluster barrier and dealloc below are warp-wide
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCtas == 2) cluster_sync();               // partner may still read our stages / signal our barriers
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}

// Self-test of the bounded wait: one thread waits on a barrier that expects two arrivals and gets one, so the wait can
// only end by running out of time (limit_ns, about a millisecond in the test).  It then does what the roles of the
// main loop do: raises the CTA's abort flag, leaves kDevTimeoutSelfTest in the status word and returns.  No tensor
// memory, no TMA, nothing in flight: the kernel always terminates and the context stays usable.
__global__ void wait_expiry_selftest_kernel(unsigned long long limit_ns, int* status, int* returned) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 2);
    fence_barrier_init();
    mbar_arrive(smem_u32(&bar));
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, kDevTimeoutSelfTest, 0, limit_ns);
    *returned = ok ? 1 : 2;     // 2: the wait gave up and the thread carried on
  }
}

}  // namespace flce
