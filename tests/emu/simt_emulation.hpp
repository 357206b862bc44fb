// A small SIMT emulation for CPU tests: runs a CUDA kernel body that uses only threadIdx / blockIdx / blockDim /
// gridDim, __shared__ arrays, __syncthreads() and full-warp shuffles on the host, one block at a time.
//
//   * every CUDA thread of a block is a fiber (ucontext) on the calling OS thread, scheduled round-robin; a barrier is a
//     generation counter that a fiber polls, yielding to the next fiber until everyone has arrived (a fiber that returns
//     from the kernel leaves the barriers, like an exited CUDA thread).  Deterministic, and no OS synchronisation;
//   * __shared__ becomes `static`: blocks run one after another, so the static storage of a kernel is the shared
//     memory of the block that is running (kernels must write it before they read it, as on the GPU);
//   * __shfl_xor_sync / __shfl_up_sync exchange through a per-block slot array and a per-warp barrier, so they need
//     all live lanes of the calling warp to take part (the kernels here call them in warp-uniform control flow only);
//   * kernels that neither synchronise nor shuffle can use launch_serial(), which runs the threads of a block in a
//     plain loop.
//
// Test infrastructure only: nothing in the library includes this file.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <vector_functions.h>
#include <vector_types.h>

#include <ucontext.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
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

struct Barrier {
  unsigned expected = 0, arrived = 0, generation = 0;
};

struct Fiber {
  ucontext_t ctx;
  std::vector<char> stack;
  bool done = false;
  Dim3 thread_idx;
};

struct BlockCtx {
  Barrier block_bar;
  std::vector<Barrier> warp_bar;
  std::vector<uint64_t> slots;
  std::vector<Fiber> fibers;
  ucontext_t scheduler;
  unsigned current = 0;
  std::function<void()> body;
};

// one OS thread: plain globals, set by the scheduler before it resumes a fiber
inline Dim3 t_thread_idx, t_block_idx;
inline BlockCtx* t_ctx = nullptr;
inline Dim3 g_block_dim, g_grid_dim;

inline unsigned linear_tid() {
  return t_thread_idx.x + g_block_dim.x * (t_thread_idx.y + g_block_dim.y * t_thread_idx.z);
}

inline void yield() {
  BlockCtx& ctx = *t_ctx;
  swapcontext(&ctx.fibers[ctx.current].ctx, &ctx.scheduler);
}

inline void barrier_release_if_complete(Barrier& b) {
  if (b.expected > 0 && b.arrived == b.expected) {
    b.arrived = 0;
    ++b.generation;
  }
}

inline void barrier_wait(Barrier& b) {
  const unsigned gen = b.generation;
  ++b.arrived;
  barrier_release_if_complete(b);
  while (b.generation == gen) yield();
}

// an exiting fiber no longer takes part: waiting fibers may now be complete
inline void barrier_drop(Barrier& b) {
  --b.expected;
  barrier_release_if_complete(b);
}

inline void fiber_entry() {
  BlockCtx& ctx = *t_ctx;
  const unsigned me = ctx.current;
  ctx.body();
  ctx.fibers[me].done = true;
  barrier_drop(ctx.block_bar);
  barrier_drop(ctx.warp_bar[me >> 5]);
  swapcontext(&ctx.fibers[me].ctx, &ctx.scheduler);      // never resumed
}

constexpr size_t kFiberStackBytes = 256 * 1024;

// the threads of a block as fibers, blocks one after another
template <typename Body>
void launch(Dim3 grid, Dim3 block, Body body) {
  g_grid_dim = grid;
  g_block_dim = block;
  const unsigned n_threads = block.x * block.y * block.z;
  BlockCtx ctx;
  ctx.body = body;
  ctx.fibers.resize(n_threads);
  for (auto& f : ctx.fibers) f.stack.resize(kFiberStackBytes);
  ctx.slots.assign(n_threads, 0);
  t_ctx = &ctx;
  for (unsigned bz = 0; bz < grid.z; ++bz)
    for (unsigned by = 0; by < grid.y; ++by)
      for (unsigned bx = 0; bx < grid.x; ++bx) {
        t_block_idx = Dim3(bx, by, bz);
        ctx.block_bar = Barrier{n_threads, 0, 0};
        ctx.warp_bar.assign((n_threads + 31) / 32, Barrier{});
        for (unsigned w = 0; w < ctx.warp_bar.size(); ++w) ctx.warp_bar[w].expected = std::min(32u, n_threads - w * 32);
        for (unsigned t = 0; t < n_threads; ++t) {
          Fiber& f = ctx.fibers[t];
          f.done = false;
          f.thread_idx = Dim3(t % block.x, (t / block.x) % block.y, t / (block.x * block.y));
          getcontext(&f.ctx);
          f.ctx.uc_stack.ss_sp = f.stack.data();
          f.ctx.uc_stack.ss_size = f.stack.size();
          f.ctx.uc_link = &ctx.scheduler;
          makecontext(&f.ctx, reinterpret_cast<void (*)()>(fiber_entry), 0);
        }
        unsigned live = n_threads;
        while (live > 0) {
          live = 0;
          for (unsigned t = 0; t < n_threads; ++t) {
            if (ctx.fibers[t].done) continue;
            ctx.current = t;
            t_thread_idx = ctx.fibers[t].thread_idx;
            swapcontext(&ctx.scheduler, &ctx.fibers[t].ctx);
            if (!ctx.fibers[t].done) ++live;
          }
        }
      }
  t_ctx = nullptr;
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
  barrier_wait(ctx.warp_bar[warp]);
  const uint64_t got = ctx.slots[warp * 32 + src_lane];
  barrier_wait(ctx.warp_bar[warp]);
  T out;
  std::memcpy(&out, &got, sizeof(T));
  return out;
}

}  // namespace emu

#define threadIdx (emu::t_thread_idx)
#define blockIdx (emu::t_block_idx)
#define blockDim (emu::g_block_dim)
#define gridDim (emu::g_grid_dim)

inline void __syncthreads() { emu::barrier_wait(emu::t_ctx->block_bar); }
// warp-level barrier: supported for blocks of exactly one warp (launch()), where it is the block barrier; a no-op
// under launch_serial(), whose kernels must not depend on it
inline void __syncwarp(unsigned = 0xffffffffu) {
  if (emu::t_ctx != nullptr) emu::barrier_wait(emu::t_ctx->block_bar);
}

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
inline float __uint_as_float(unsigned v) {
  float f;
  std::memcpy(&f, &v, sizeof(f));
  return f;
}
inline unsigned __float_as_uint(float f) {
  unsigned v;
  std::memcpy(&v, &f, sizeof(v));
  return v;
}

using std::max;
using std::min;
