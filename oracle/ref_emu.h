// CUDA-on-the-host emulation, just wide enough to run the reference's own kernels (its .cu sources) on
// a CPU, one emulated thread at a time.  TEST INFRASTRUCTURE: it exists so that the parity oracle can be
// checked against the reference's kernels in a container without a GPU; nothing the library ships
// includes it.
//
// How a launch runs: the build recipe (build_ref.py) rewrites `kernel<<<grid, block[, shmem]>>>(args)` into
// `REF_EMU_LAUNCH(grid, block, shmem, kernel(args))`.  Blocks run one after another; the threads of a block
// are fibers (ucontext) on one OS thread, resumed round-robin, and `__syncthreads()` yields to the scheduler,
// so every fiber reaches barrier r before any continues to barrier r+1 -- the semantics kernels with
// shared-memory staging rely on.  `__shared__` arrays are statics (blocks never overlap in time), device
// memory is host memory (cudaMalloc = malloc), atomics are plain read-modify-writes (one OS thread).
#pragma once
#include <ucontext.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <vector>

struct uint2 { unsigned int x, y; };
struct uint3 { unsigned int x, y, z; };
struct int2 { int x, y; };
struct float2 { float x, y; };
struct dim3 {
  unsigned int x, y, z;
  dim3(unsigned int x_ = 1, unsigned int y_ = 1, unsigned int z_ = 1) : x(x_), y(y_), z(z_) {}
};
static uint3 threadIdx, blockIdx;
static dim3 blockDim, gridDim;

#define __global__
#define __device__
#define __host__
#define __constant__
#define __forceinline__ inline
#define __restrict__
#define __shared__ static
#define __launch_bounds__(...)

namespace ref_emu {
struct Fiber {
  ucontext_t ctx;
  bool done = false;
};
static ucontext_t g_sched;
static Fiber *g_current = nullptr;
static const std::function<void()> *g_body = nullptr;
static void trampoline() {
  (*g_body)();
  g_current->done = true;
  swapcontext(&g_current->ctx, &g_sched);
}
inline void sync_threads() { swapcontext(&g_current->ctx, &g_sched); }

inline void launch(dim3 grid, dim3 block, const std::function<void()> &body) {
  const size_t nthreads = (size_t)block.x * block.y * block.z;
  const size_t stack_bytes = 256 * 1024;
  static std::vector<char> stacks;
  if (stacks.size() < nthreads * stack_bytes) stacks.resize(nthreads * stack_bytes);
  std::vector<Fiber> fibers(nthreads);
  gridDim = grid;
  blockDim = block;
  g_body = &body;
  for (unsigned bz = 0; bz < grid.z; ++bz)
    for (unsigned by = 0; by < grid.y; ++by)
      for (unsigned bx = 0; bx < grid.x; ++bx) {
        for (size_t t = 0; t < nthreads; ++t) {
          Fiber &f = fibers[t];
          f.done = false;
          getcontext(&f.ctx);
          f.ctx.uc_stack.ss_sp = stacks.data() + t * stack_bytes;
          f.ctx.uc_stack.ss_size = stack_bytes;
          f.ctx.uc_link = nullptr;
          makecontext(&f.ctx, trampoline, 0);
        }
        size_t live = nthreads;
        while (live) {  // one round = every live thread runs up to its next barrier (or to its end)
          live = 0;
          for (size_t t = 0; t < nthreads; ++t) {
            Fiber &f = fibers[t];
            if (f.done) continue;
            blockIdx = uint3{bx, by, bz};
            threadIdx = uint3{(unsigned)(t % block.x), (unsigned)((t / block.x) % block.y),
                              (unsigned)(t / ((size_t)block.x * block.y))};
            g_current = &f;
            swapcontext(&g_sched, &f.ctx);
            if (!f.done) ++live;
          }
        }
      }
  g_body = nullptr;
}
}  // namespace ref_emu

#define REF_EMU_LAUNCH(grid, block, shmem, call) ref_emu::launch(dim3(grid), dim3(block), [&]() { call; })
#define __syncthreads() ref_emu::sync_threads()

// ---- the slice of the runtime API the reference's host code calls: device memory is host memory ----
typedef int cudaError_t;
typedef void *cudaStream_t;
enum { cudaSuccess = 0 };
enum cudaMemcpyKind { cudaMemcpyHostToHost, cudaMemcpyHostToDevice, cudaMemcpyDeviceToHost, cudaMemcpyDeviceToDevice };
inline const char *cudaGetErrorString(cudaError_t) { return "emulated"; }
inline cudaError_t cudaGetLastError() { return cudaSuccess; }
inline cudaError_t cudaPeekAtLastError() { return cudaSuccess; }
inline cudaError_t cudaDeviceSynchronize() { return cudaSuccess; }
template <class T> inline cudaError_t cudaMalloc(T **p, size_t bytes) {
  *p = static_cast<T *>(std::malloc(bytes ? bytes : 1));
  return cudaSuccess;
}
inline cudaError_t cudaFree(void *p) {
  std::free(p);
  return cudaSuccess;
}
inline cudaError_t cudaMemcpy(void *d, const void *s, size_t n, cudaMemcpyKind) {
  std::memmove(d, s, n);
  return cudaSuccess;
}
inline cudaError_t cudaMemset(void *d, int v, size_t n) {
  std::memset(d, v, n);
  return cudaSuccess;
}

// ---- device intrinsics used by the kernels ----
template <class T, class U> inline T atomicAdd(T *p, U v) {
  T old = *p;
  *p = old + (T)v;
  return old;
}
template <class T> inline T atomicCAS(T *p, T cmp, T v) {
  T old = *p;
  if (old == cmp) *p = v;
  return old;
}
template <class T> inline T atomicExch(T *p, T v) {
  T old = *p;
  *p = v;
  return old;
}
template <class T> inline T atomicMax(T *p, T v) {
  T old = *p;
  if (v > old) *p = v;
  return old;
}
template <class T> inline T __ldg(const T *p) { return *p; }
inline float __fmaf_rn(float a, float b, float c) { return std::fmaf(a, b, c); }
