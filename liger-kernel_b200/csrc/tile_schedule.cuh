// Tile geometry and the static tile schedule of the tcgen05 main loop (gemm_sm100.cuh): which (m-tile, n-tile) a
// persistent CTA (or CTA pair) works on at each step, and how a device-resident count of rows that matter shrinks the
// work.  Pure integer arithmetic, shared by the three warp roles of the kernel (they must agree tile for tile) and
// compiled for the host by the CPU tests.
#pragma once

namespace flce {

constexpr int kBlockM = 128;      // rows per CTA
constexpr int kBlockN = 256;      // columns per tile
constexpr int kBlockK = 64;       // two-byte elements per stage = one 128-byte swizzle row

struct GemmShape {
  int M, N, K;         // logical extents
  int m_tiles;         // ceil(M / (128 * kCtas))
  int n_tiles;         // ceil(N / 256)
  int k_blocks;        // ceil(K / 64)
  int group;           // raster: tiles are walked in groups of `group` rows (or columns) of tiles
  int group_along_m;   // 1: a group is `group` m-tiles x all n-tiles, m fastest; 0: the transpose
  int hint_a, hint_b;  // L2 eviction priority of the A / B loads: 0 default, 1 evict first, 2 evict last
  int poll_sleep_ns;   // back-off of the epilogue warps while they wait for an accumulator
  // Optional device-resident row count (rows that matter come first, e.g. after ignored tokens were moved to the end):
  // role 1 limits the m-tiles to those that contain such rows, role 2 limits the k-blocks (when K runs over rows).
  // active_base is the index of this launch's first row in the numbering active_rows counts in (a token chunk).
  const int* active_rows;
  int active_role;
  int active_base;
  // Optional device-resident switch: when it points at 0 the whole launch returns at once (a pass that only some
  // inputs need is enqueued unconditionally and decides on the device, without a host synchronisation).
  const int* gate;
  // Per cent of a tile's K range over which the units' first tiles are cut in two at unit-dependent points (0 = never).
  // All units of a persistent grid otherwise finish their equally long tiles at the same moment, and their epilogues
  // (fp32 read-modify-write of the whole output wave) hit memory as one burst while every tensor core waits.
  int stagger;
};

// k-block at which unit `unit` cuts its first tile (0: not cut)
__device__ __forceinline__ int stagger_split(const GemmShape& s, int unit, int num_units) {
  if (s.stagger <= 0 || s.k_blocks < 16 || num_units < 2) return 0;
  const long long span = static_cast<long long>(s.k_blocks) * s.stagger / 100;
  const int cut = 1 + static_cast<int>(span * (2 * unit + 1) / (2 * num_units));
  return cut < s.k_blocks ? cut : s.k_blocks - 1;
}

__device__ __forceinline__ void decode_tile(const GemmShape& s, int tile, int& mt, int& nt) {
  if (s.group_along_m) {
    const int per_group = s.group * s.n_tiles;
    const int g = tile / per_group;
    const int r = tile - g * per_group;
    const int first = g * s.group;
    const int rows = min(s.group, s.m_tiles - first);
    nt = r / rows;
    mt = first + (r - nt * rows);
  } else {
    const int per_group = s.group * s.m_tiles;
    const int g = tile / per_group;
    const int r = tile - g * per_group;
    const int first = g * s.group;
    const int cols = min(s.group, s.n_tiles - first);
    mt = r / cols;
    nt = first + (r - mt * cols);
  }
}


// rows that matter come first: role 1 drops the m-tiles behind them, role 2 the k-blocks (K runs over rows)
__device__ __forceinline__ void limit_to_active_rows(GemmShape& shape, int active_rows, int ctas_per_tile) {
  const int rows = max(0, active_rows);
  if (shape.active_role == 1)
    shape.m_tiles = min(shape.m_tiles, (rows + kBlockM * ctas_per_tile - 1) / (kBlockM * ctas_per_tile));
  else if (shape.active_role == 2)
    shape.k_blocks = min(shape.k_blocks, (rows + kBlockK - 1) / kBlockK);
}

}  // namespace flce
