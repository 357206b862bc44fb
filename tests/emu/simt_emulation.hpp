// A small SIMT emulation for CPU tests: runs a CUDA kernel body that uses only threadIdx / blockIdx / blockDim /
// gridDim, __shared__ arrays, __syncthreads() and full-warp shuffles on host threads, one block at a time.
//
//   * every CUDA thread of a block is one std::thread; __syncthreads() is a std::barrier over the block's threads
//     (a thread that returns from the kernel leaves the barrier, like an exited CUDA thread);
//   * __shared__ becomes `static`: blocks run one after another, so the static storage of a kernel is the shared
//     memory of the block that is running (kernels must write it before they read it, as on the GPU);
//   * __shfl_xor_sync / __shfl_up_sync exchange through a per-block slot array and a per-warp barrier, so they need
//     all 32 lanes of the calling warp to take part (the kernels here call them in warp-uniform control flow only);
//   * kernels that neither synchronise nor shuffle can use launch_serial(), which runs the threads of a block in a
//     plain loop.
//
// Test infrastructure only: nothing in the library includes this file.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <vector_functions.h>
#include <vector_types.h>

#include <algorithm>
#include <barrier>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

#undef __shared__
#define __shared__ static
#undef __launch_bounds__
#define __launch_bounds__(...)
#undef __global__
#define __global__
#undef __device__
#define __device__
#undef __host__
#define __host__
#undef __forceinline__
#define __forceinline__ inline

namespace emu {

struct Dim3 {
  unsigned x = 1, y = 1, z = 1;
  Dim3() = default;
  Dim3(unsigned x_, unsigned y_ = 1, unsigned z_ = 1) : x(x_), y(y_), z(z_) {}
};

struct BlockCtx {
  explicit BlockCtx(unsigned n_threads)
      : block_bar(static_cast<std::ptrdiff_t>(n_threads)), slots(n_threads, 0) {
    for (unsigned w = 0; w < (n_threads + 31) / 32; ++w) {
      const unsigned lanes = std::min(32u, n_threads - w * 32);
      warp_bar.emplace_back(std::make_unique<std::barrier<>>(static_cast<std::ptrdiff_t>(lanes)));
    }
  }
  std::barrier<> block_bar;
  std::vector<std::unique_ptr<std::barrier<>>> warp_bar;
  std::vector<uint64_t> slots;
};

inline thread_local Dim3 t_thread_idx, t_block_idx;
inline thread_local BlockCtx* t_ctx = nullptr;
inline Dim3 g_block_dim, g_grid_dim;

inline unsigned linear_tid() {
  return t_thread_idx.x + g_block_dim.x * (t_thread_idx.y + g_block_dim.y * t_thread_idx.z);
}

// one std::thread per CUDA thread, blocks one after another
template <typename Body>
void launch(Dim3 grid, Dim3 block, Body body) {
  g_grid_dim = grid;
  g_block_dim = block;
  const unsigned n_threads = block.x * block.y * block.z;
  for (unsigned bz = 0; bz < grid.z; ++bz)
    for (unsigned by = 0; by < grid.y; ++by)
      for (unsigned bx = 0; bx < grid.x; ++bx) {
        BlockCtx ctx(n_threads);
        std::vector<std::thread> threads;
        threads.reserve(n_threads);
        for (unsigned t = 0; t < n_threads; ++t) {
          threads.emplace_back([&, t]() {
            t_ctx = &ctx;
            t_block_idx = Dim3(bx, by, bz);
            t_thread_idx = Dim3(t % block.x, (t / block.x) % block.y, t / (block.x * block.y));
            body();
            ctx.block_bar.arrive_and_drop();
          });
        }
        for (auto& th : threads) th.join();
      }
}

// for kernels without __syncthreads() and shuffles
template <typename Body>
void launch_serial(Dim3 grid, Dim3 block, Body body) {
  g_grid_dim = grid;
  g_block_dim = block;
  t_ctx = nullptr;
  for (unsigned bz = 0; bz < grid.z; ++bz)
    for (unsigned by = 0; by < grid.y; ++by)
      for (unsigned bx = 0; bx < grid.x; ++bx)
        for (unsigned tz = 0; tz < block.z; ++tz)
          for (unsigned ty = 0; ty < block.y; ++ty)
            for (unsigned tx = 0; tx < block.x; ++tx) {
              t_block_idx = Dim3(bx, by, bz);
              t_thread_idx = Dim3(tx, ty, tz);
              body();
            }
}

template <typename T>
T shuffle_from(T v, unsigned src_lane) {
  static_assert(sizeof(T) <= 8, "shuffles move at most 8 bytes");
  BlockCtx& ctx = *t_ctx;
  const unsigned tid = linear_tid(), warp = tid >> 5;
  uint64_t bits = 0;
  std::memcpy(&bits, &v, sizeof(T));
  ctx.slots[tid] = bits;
  ctx.warp_bar[warp]->arrive_and_wait();
  const uint64_t got = ctx.slots[warp * 32 + src_lane];
  ctx.warp_bar[warp]->arrive_and_wait();
  T out;
  std::memcpy(&out, &got, sizeof(T));
  return out;
}

}  // namespace emu

#define threadIdx (emu::t_thread_idx)
#define blockIdx (emu::t_block_idx)
#define blockDim (emu::g_block_dim)
#define gridDim (emu::g_grid_dim)

inline void __syncthreads() { emu::t_ctx->block_bar.arrive_and_wait(); }

template <typename T>
T __shfl_xor_sync(unsigned, T v, int lane_mask) {
  return emu::shuffle_from(v, (emu::linear_tid() & 31u) ^ static_cast<unsigned>(lane_mask));
}
template <typename T>
T __shfl_up_sync(unsigned, T v, unsigned delta) {
  const unsigned lane = emu::linear_tid() & 31u;
  return emu::shuffle_from(v, lane >= delta ? lane - delta : lane);
}
template <typename T>
T __ldg(const T* p) { return *p; }

using std::max;
using std::min;
